"""Child process of test_dependent_launch_changes_nothing: runs a chain of MoE
blocks (each layer consumes the previous layer's output, so every kernel
depends on the one before it) and prints a digest of all layer outputs."""
import hashlib
import sys

import torch


def main():
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    dev = torch.device("cuda:0")
    torch.manual_seed(1234)
    blocks = []
    for i in range(6):
        blk = SparseMoeBlock(1152, 4, 8, 2, pretraining_tp=1, layer_idx=i, total_layers=6, para_mode=ParaMode(),
                             expert_act="gelu_tanh", shared_expert=False)
        blk.gate.norm_topk_prob = True
        for p in blk.parameters():
            torch.nn.init.normal_(p, std=0.02)
        blocks.append(blk.to(device=dev, dtype=torch.bfloat16).eval())
    x = torch.randn(8, 256, 1152, device=dev).bfloat16()
    digest = hashlib.sha256()
    with torch.no_grad():
        for rep in range(3):
            h = x
            for blk in blocks:
                h = (h + blk(h)).contiguous()
                digest.update(h.float().cpu().numpy().tobytes())
    for blk in blocks:
        blk.check_status()
    print("DIGEST", digest.hexdigest())


if __name__ == "__main__":
    sys.exit(main())
