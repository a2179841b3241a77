"""A chain of MoE blocks captured into one CUDA graph (dice_b200.serving.GraphedStep) replays to the same bits
as the eager calls, for new inputs too; expert-parallel blocks are refused."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant", ["gelu_tanh", "swiglu"])
def test_graphed_chain_of_blocks_equals_eager(cuda_device, variant):
    from dice_b200.moe_block import ParaMode, SparseMoeBlock
    from dice_b200.serving import GraphedStep

    torch.manual_seed(3)
    h, e, layers = 256, 8, 3
    blocks = []
    for layer in range(layers):
        blk = SparseMoeBlock(h, 4, e, 2, 1, layer, layers, ParaMode(), expert_act=variant,
                             shared_expert=(variant == "swiglu"))
        blk.gate.norm_topk_prob = variant == "gelu_tanh"
        blocks.append(blk.to(device=cuda_device, dtype=torch.bfloat16).eval())

    def chain(x):
        for blk in blocks:
            x = x + blk(x)
        return x

    g = torch.Generator(device="cuda").manual_seed(4)
    xs = [torch.randn(2, 300, h, generator=g, device=cuda_device).bfloat16() for _ in range(3)]
    want = [chain(x) for x in xs]
    step = GraphedStep(chain, xs[0], modules=blocks)
    for x, w in zip(xs, want):
        got = step(x)
        torch.cuda.synchronize()
        assert torch.equal(got, w)
    for blk in blocks:
        blk.check_status()


def test_expert_parallel_blocks_are_refused(cuda_device):
    from dice_b200.serving import GraphedStep

    class Fake(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.para_mode = type("P", (), {"ep": True})()

    with pytest.raises(RuntimeError, match="expert-parallel"):
        GraphedStep(lambda x: x, torch.zeros(1, device=cuda_device), modules=[Fake()])
