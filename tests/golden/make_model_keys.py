"""Generate tests/golden/convnext_keys.json and backbone_keys.json: the state-dict keys and
shapes of the REFERENCE's classifier models (models/convnext.py) and of its dense-prediction
backbone (semantic_segmentation/backbone/convnext.py), for the checkpoint-layout tests.

Needs the reference checkout; imports both files unmodified behind stand-ins for the packages
this image lacks — three `timm` names (trunc_normal_, DropPath, register_model) and, for the
backbone, `mmcv_custom.load_checkpoint`, `mmseg.utils.get_root_logger` and a `BACKBONES`
registry — and with this repository's operator module answering `import dwoconv1d`.

    python tests/golden/make_model_keys.py
"""
import json
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.build import reference_root  # noqa: E402

REF = reference_root()
if REF is None:
    raise SystemExit("no reference checkout (set O1D_REFERENCE_ROOT)")
sys.path.insert(0, ROOT)

import oriented1d_b200  # noqa: E402

sys.path.insert(0, oriented1d_b200.compat_path())
timm = types.ModuleType("timm")
models = types.ModuleType("timm.models")
layers = types.ModuleType("timm.models.layers")
registry = types.ModuleType("timm.models.registry")
layers.trunc_normal_ = torch.nn.init.trunc_normal_


class DropPath(torch.nn.Module):
    def __init__(self, p=0.0):
        super().__init__()
        self.p = p

    def forward(self, x):
        return x


layers.DropPath = DropPath
registry.register_model = lambda f: f
sys.modules.update({"timm": timm, "timm.models": models, "timm.models.layers": layers,
                    "timm.models.registry": registry})
sys.path.insert(0, REF)
from models import convnext as ref  # noqa: E402

out = {}
for name, factory, variant in (("tiny_1d", ref.convnext_tiny, "1d"), ("tiny_1dpp", ref.convnext_tiny, "1dpp"),
                               ("base_1dpp", ref.convnext_base, "1dpp"), ("tiny_2dpp", ref.convnext_tiny, "2dpp"),
                               ("tiny_2d", ref.convnext_tiny, "2d")):
    m = factory(variant=variant)
    out[name] = {k: list(v.shape) for k, v in m.state_dict().items()}
    out[name + "_params"] = sum(p.numel() for p in m.parameters())
    # per-layer angle lists: the rasterised lines depend on them
    out[name + "_theta_sample"] = {k: [float(x) for x in v.flatten()[:16]] for k, v in m.state_dict().items()
                                   if k.endswith("theta") and ("stages.0.0" in k or "stages.0.1" in k or "dw1" in k)}
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "convnext_keys.json")
json.dump(out, open(path, "w"))
print(path, os.path.getsize(path), {k: v for k, v in out.items() if k.endswith("_params")})


# ---- dense-prediction backbone -----------------------------------------------------------------------
import importlib.util  # noqa: E402

mmcv_custom = types.ModuleType("mmcv_custom")
mmcv_custom.load_checkpoint = lambda *a, **k: None
mmseg = types.ModuleType("mmseg")
mmseg_utils = types.ModuleType("mmseg.utils")
mmseg_utils.get_root_logger = lambda *a, **k: None
mmseg_models = types.ModuleType("mmseg.models")
mmseg_builder = types.ModuleType("mmseg.models.builder")


class _Registry:
    def register_module(self):
        return lambda cls: cls


mmseg_builder.BACKBONES = _Registry()
sys.modules.update({"mmcv_custom": mmcv_custom, "mmseg": mmseg, "mmseg.utils": mmseg_utils,
                    "mmseg.models": mmseg_models, "mmseg.models.builder": mmseg_builder})
spec = importlib.util.spec_from_file_location(
    "ref_backbone", os.path.join(REF, "semantic_segmentation", "backbone", "convnext.py"))
refbb = importlib.util.module_from_spec(spec)
spec.loader.exec_module(refbb)

bb = {}
for name, kw in (("tiny_1d", dict(variant="1d")), ("tiny_1dpp", dict(variant="1dpp")),
                 ("tiny_2dpp", dict(variant="2dpp")),
                 ("base_1dpp", dict(variant="1dpp", depths=[3, 3, 27, 3], dims=[128, 256, 512, 1024]))):
    m = refbb.ConvNeXt(**kw)
    bb[name] = {k: list(v.shape) for k, v in m.state_dict().items()}
    bb[name + "_params"] = sum(p.numel() for p in m.parameters())
    bb[name + "_theta_sample"] = {k: [float(x) for x in v.flatten()[:16]] for k, v in m.state_dict().items()
                                  if k.endswith("theta") and ("stages.2.1" in k or "stages.3.0" in k or "dw2" in k)}
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "backbone_keys.json")
json.dump(bb, open(path, "w"))
print(path, os.path.getsize(path), {k: v for k, v in bb.items() if k.endswith("_params")})
