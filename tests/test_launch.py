"""The launcher installs this package's modules over the reference's (needs
the reference checkout; skipped elsewhere)."""
import subprocess
import sys
import textwrap

import pytest

from oracle.reference_shim import DEFAULT_REFERENCE_ROOT, reference_available


@pytest.mark.skipif(not reference_available(), reason="reference checkout not present")
def test_install_replaces_reference_modules():
    code = textwrap.dedent(
        f"""
        import sys
        sys.path.insert(0, {repr(sys.path[0])})
        from oracle.reference_shim import load_reference  # registers the timm stub
        import types, torch.nn as nn
        timm = types.ModuleType("timm"); tm = types.ModuleType("timm.models"); vit = types.ModuleType("timm.models.vision_transformer")
        for n in ("PatchEmbed", "Attention", "Mlp"):
            setattr(vit, n, type(n, (nn.Module,), {{}}))
        sys.modules.update({{"timm": timm, "timm.models": tm, "timm.models.vision_transformer": vit}})
        from dice_b200 import launch, moe_block
        models = launch.install({repr(DEFAULT_REFERENCE_ROOT)})
        assert models.SparseMoeBlock is moe_block.SparseMoeBlock
        from expertpara.diep import ep_cache_init, ep_set_step
        from expertpara.ep_fwd import moe_infer_ep, use_latest_expert_weights
        from expertpara.etrim import trim_state_dict
        import dice_b200.expertpara.diep as mine
        assert ep_cache_init is mine.ep_cache_init
        # the reference's own sampler-side imports resolve to the replacements
        import diffusion.rectified_flow as rf
        assert rf.ep_set_step is mine.ep_set_step
        # DiTBlock's lookup of SparseMoeBlock goes through the patched module global
        assert models.DiTBlock.__init__.__globals__["SparseMoeBlock"] is moe_block.SparseMoeBlock
        print("ok")
        """
    )
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
