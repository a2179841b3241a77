"""Run an unmodified DICE script on the dice_b200 MoE block.

    cd /path/to/DICE
    torchrun --nproc_per_node 8 -m dice_b200.launch sample_ddp.py --model DiT-XL/2 --ep --ep-async ...

``install()`` puts this package's modules in the place of the reference's
``expertpara.{ep_fwd,diep,ep_cache,etrim}`` (before anything imports names
from them) and its ``SparseMoeBlock`` / ``MoEGate`` / ``MoeMLP`` in the place
of the classes of the reference's ``models`` module, which ``DiTBlock`` looks
up by name when it builds a block (models.py:498-507), and lets
``DiTBlock.forward`` hand the LayerNorm + modulation in front of the MoE block
and the gated residual behind it to the block's kernels.  Everything else of
the reference (DiT backbone, attention, samplers, flags, state-dict loading)
runs as is.
"""
from __future__ import annotations

import contextlib
import importlib
import os
import runpy
import sys


def _ditblock_forward(self, x, c):
    """``DiTBlock.forward`` (models.py:514-520) with its MoE half handed to
    ``SparseMoeBlock.forward_with_glue``: the attention half is the
    reference's, the LayerNorm + modulation in front of the MoE block and the
    gated residual behind it run inside this package's kernels."""
    from .expertpara import diep

    prof = diep._profiler()
    scope = prof.scope if prof is not None else (lambda name: contextlib.nullcontext())
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = self.adaLN_modulation(c).chunk(6, dim=1)
    with scope("attn"):
        normed = self.norm1(x)
        x = x + gate_msa.unsqueeze(1) * self.attn(normed * (1 + scale_msa.unsqueeze(1)) + shift_msa.unsqueeze(1))
    with scope("moe"):
        return self.moe.forward_with_glue(x, shift_mlp, scale_mlp, gate_mlp, eps=self.norm2.eps)


def install(reference_root: str | None = None):
    """Patch the reference's modules in ``sys.modules``; returns its ``models`` module."""
    root = os.path.abspath(reference_root or os.getcwd())
    if not os.path.isfile(os.path.join(root, "models.py")):
        raise FileNotFoundError(f"{root} does not look like a DICE checkout (models.py not found)")
    if root not in sys.path:
        sys.path.insert(0, root)
    from . import expertpara as mine
    from .expertpara import diep, ep_cache, ep_fwd, etrim

    ref_pkg = importlib.import_module("expertpara")
    if os.path.abspath(os.path.dirname(ref_pkg.__file__)) == os.path.abspath(os.path.dirname(mine.__file__)):
        raise RuntimeError("the name 'expertpara' resolved to dice_b200's own package; run from the DICE checkout")
    for name, mod in (("ep_fwd", ep_fwd), ("diep", diep), ("ep_cache", ep_cache), ("etrim", etrim)):
        sys.modules[f"expertpara.{name}"] = mod
        setattr(ref_pkg, name, mod)
    models = importlib.import_module("models")
    from . import moe_block

    models.SparseMoeBlock = moe_block.SparseMoeBlock
    models.MoEGate = moe_block.MoEGate
    models.MoeMLP = moe_block.MoeMLP
    models.trim_module_list = etrim.trim_module_list
    # the element-wise glue around the MoE block moves into its kernels unless DICE_FUSED_GLUE=0
    if os.environ.get("DICE_FUSED_GLUE", "1") != "0":
        models.DiTBlock.forward = _ditblock_forward
    # expert parallelism exchanges rows over NVLink peer memory unless DICE_EP_P2P=0 (NCCL is the fallback
    # when peer memory cannot be mapped)
    if os.environ.get("DICE_EP_P2P", "1") != "0":
        from .expertpara import p2p

        # a sampling script's ranks may stall for seconds between two model calls (saving images, logging):
        # the exchange kernels wait 30 s for a peer here instead of their 2 s default (the reference's
        # collectives wait for the process group's timeout)
        os.environ.setdefault("DICE_EP_P2P_WAIT_MS", "30000")
        p2p.enable(True)
    return models


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit("usage: python -m dice_b200.launch <script.py> [script arguments]")
    script = argv[0]
    install(os.path.dirname(os.path.abspath(script)) or None)
    sys.argv = argv
    runpy.run_path(script, run_name="__main__")


if __name__ == "__main__":
    main()
