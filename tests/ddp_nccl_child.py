"""Child process of test_nccl_data_parallel_matches_single_process (one per GPU, via torchrun)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F


def main():
    out_dir = sys.argv[1]
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    from snn_gpu_training_bptt_b200.example import models
    from snn_gpu_training_bptt_b200.example.ddp import DistributedDataParallel

    def make():
        torch.manual_seed(11)
        return models.SpikingVGG(time_steps=4, widths=(8, 16, 16), hidden=32, image=16,
                                 act_dtype=torch.float32).to(dev)

    gen = torch.Generator().manual_seed(5)
    images = torch.rand((4 * world, 3, 16, 16), generator=gen).to(dev)
    labels = torch.randint(0, 10, (4 * world,), generator=gen).to(dev)

    net = make()
    ddp = DistributedDataParallel(net, bucket_mb=0.01)
    ddp.zero_grad()
    sl = slice(4 * rank, 4 * rank + 4)
    F.cross_entropy(ddp(images[sl]), labels[sl]).backward()
    torch.cuda.synchronize()
    torch.save({n: p.grad.cpu() for n, p in net.named_parameters()}, os.path.join(out_dir, f"rank{rank}.pt"))
    if rank == 0:
        ref = make()
        F.cross_entropy(ref(images), labels).backward()
        torch.save({n: p.grad.cpu() for n, p in ref.named_parameters()}, os.path.join(out_dir, "single.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
