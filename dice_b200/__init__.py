"""dice_b200: the DiT-MoE sparse MoE block and its expert-parallel exchange on
NVIDIA B200 (sm_100a) kernels, behind the module interface of DICE.

``SparseMoeBlock`` / ``MoEGate`` / ``MoeMLP`` / ``ParaMode`` mirror the
reference's ``models.py``; ``dice_b200.expertpara`` mirrors its ``expertpara``
package (``ep_fwd``, ``diep``, ``ep_cache``, ``etrim``).  The compute runs in
``libdice_b200.so`` (C ABI declared in ``include/dice_b200.h``); importing the
package does not need a GPU, running a block does.
"""

__all__ = ["SparseMoeBlock", "MoEGate", "MoeMLP", "GeluMLP", "ParaMode", "ops"]


def __getattr__(name):
    if name in ("SparseMoeBlock", "MoEGate", "MoeMLP", "GeluMLP", "ParaMode", "ExpertPack", "layer_is_async"):
        from . import moe_block

        return getattr(moe_block, name)
    if name == "ops":
        import importlib

        return importlib.import_module(".ops", __name__)
    raise AttributeError(name)
