"""Child process of test_sync_bn_layers_over_nccl (one per GPU, launched by torchrun)."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    out_dir = sys.argv[1]
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    from snn_gpu_training_bptt_b200 import snnlib_op as sop

    gen = torch.Generator().manual_seed(3)
    x = (torch.randn((6, 4, 8, 6, 6), generator=gen) * 1.2 + 0.1).to(dev)
    xf = (torch.randn((6, 4, 8), generator=gen) * 1.2 + 0.1).to(dev)
    gy_conv = torch.randn((6, 4, 8, 6, 6), generator=gen).to(dev)
    gy_fc = torch.randn((6, 4, 5), generator=gen).to(dev)
    gy_bn = torch.randn((6, 4, 8), generator=gen).to(dev)

    def build(dist_mode):
        torch.manual_seed(5)
        conv = (sop.BnFireConvDist if dist_mode else sop.BnFireConv)(8, 8).to(dev)
        torch.manual_seed(6)
        fc = (sop.BnFireFcDist if dist_mode else sop.BnFireFc)(8, 5, (0, 1)).to(dev)
        bn = (sop.BnDist if dist_mode else sop.Bn)(8, (0, 1)).to(dev)
        for m in (conv, fc, bn):
            with torch.no_grad():
                m.weight_bn.copy_(torch.linspace(0.6, 1.4, 8))
                m.bias_bn.copy_(torch.linspace(-0.2, 0.3, 8))
        return conv, fc, bn

    def run(mods, sl):
        conv, fc, bn = mods
        res = {}
        xi = x[:, sl].contiguous().requires_grad_(True)
        y = conv(xi); y.backward(gy_conv[:, sl].contiguous())
        res["y_conv"], res["gx_conv"] = y.detach().cpu(), xi.grad.cpu()
        res["gwbn_conv"], res["gw_conv"] = conv.weight_bn.grad.cpu(), conv.weight_conv.grad.cpu()
        xi = xf[:, sl].contiguous().requires_grad_(True)
        y = fc(xi); y.backward(gy_fc[:, sl].contiguous())
        res["y_fc"], res["gx_fc"] = y.detach().cpu(), xi.grad.cpu()
        res["gbbn_fc"], res["gw_fc"] = fc.bias_bn.grad.cpu(), fc.weight_fc.grad.cpu()
        xi = xf[:, sl].contiguous().requires_grad_(True)
        y = bn(xi); y.backward(gy_bn[:, sl].contiguous())
        res["y_bn"], res["gx_bn"], res["gwbn_bn"] = y.detach().cpu(), xi.grad.cpu(), bn.weight_bn.grad.cpu()
        return res

    res = run(build(True), slice(2 * rank, 2 * rank + 2))
    # the same sync-BN layers on bf16 activations: statistics are all-reduced in fp32
    conv16, fc16, _ = build(True)
    xi = x[:, 2 * rank:2 * rank + 2].contiguous().to(torch.bfloat16).requires_grad_(True)
    y16 = conv16(xi)
    y16.backward(gy_conv[:, 2 * rank:2 * rank + 2].contiguous().to(torch.bfloat16))
    res["bf16_y_conv"], res["bf16_gx_conv"] = y16.detach().float().cpu(), xi.grad.float().cpu()
    res["bf16_running_var"] = conv16.running_var.detach().cpu()
    torch.save(res, os.path.join(out_dir, f"rank{rank}.pt"))
    if rank == 0:
        torch.save(run(build(False), slice(0, 4)), os.path.join(out_dir, "single.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
