"""Import the unmodified reference (DICE) Python modules for oracle validation.

Test infrastructure only.  Used on a machine that has the reference checkout
(to validate ``oracle.moe_oracle`` and to generate the fixtures committed under
``tests/golden``); it is never needed at run time of the product, of the GPU
tests or of the benchmark.

Two shims are required and neither edits the reference's sources:

* ``models.py:16`` imports ``timm.models.vision_transformer`` at module load;
  ``timm`` is not installed, so placeholder classes are registered (only the
  MoE classes of ``models.py`` are used by the oracle).
* the hot path enters ``CudaProfiler.scope`` (``models.py:305``,
  ``expertpara/ep_fwd.py:88`` ...), which records CUDA events
  (``cudaprof/prof.py:22-26``); without a CUDA driver that raises, so the
  scope is replaced by a null context manager.
"""
import contextlib
import os
import sys
import types

# the reference checkout: $DICE_REFERENCE_ROOT, else a directory "reference" next to this repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_REFERENCE_ROOT = os.environ.get("DICE_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO), "reference"))


def reference_available(root: str = DEFAULT_REFERENCE_ROOT) -> bool:
    return os.path.isfile(os.path.join(root, "models.py"))


def load_reference(root: str = DEFAULT_REFERENCE_ROOT):
    """Return a namespace with the reference's ``models``, ``ep_fwd``, ``diep``,
    ``ep_cache`` and ``etrim`` modules imported from ``root``."""
    if not reference_available(root):
        raise FileNotFoundError(f"reference checkout not found at {root}")
    if "timm" not in sys.modules:
        import torch.nn as nn

        timm = types.ModuleType("timm")
        timm_models = types.ModuleType("timm.models")
        vit = types.ModuleType("timm.models.vision_transformer")
        for name in ("PatchEmbed", "Attention", "Mlp"):
            setattr(vit, name, type(name, (nn.Module,), {}))
        timm.models = timm_models
        timm_models.vision_transformer = vit
        sys.modules["timm"] = timm
        sys.modules["timm.models"] = timm_models
        sys.modules["timm.models.vision_transformer"] = vit
    if root not in sys.path:
        sys.path.insert(0, root)
    import torch

    from cudaprof.prof import CudaProfiler

    if not torch.cuda.is_available():

        @contextlib.contextmanager
        def _null_scope(name, stream=None, cpu=False):
            yield

        CudaProfiler.scope = staticmethod(_null_scope)

    import models  # noqa: E402  (the reference's models.py)
    from expertpara import diep, ep_cache, ep_fwd, etrim  # noqa: E402

    return types.SimpleNamespace(
        models=models, ep_fwd=ep_fwd, diep=diep, ep_cache=ep_cache, etrim=etrim
    )
