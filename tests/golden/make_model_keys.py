"""Generate tests/golden/convnext_keys.json: the state-dict keys and shapes of the
REFERENCE's ConvNeXt-1D / 1D++ models (models/convnext.py), for the checkpoint-layout test.

Needs the reference checkout; imports its models/convnext.py unmodified behind a three-name
`timm` stand-in (trunc_normal_, DropPath, register_model) and with this repository's operator
module answering `import dwoconv1d`.

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
                               ("base_1dpp", ref.convnext_base, "1dpp")):
    m = factory(variant=variant)
    out[name] = {k: list(v.shape) for k, v in m.state_dict().items()}
    out[name + "_params"] = sum(p.numel() for p in m.parameters())
    # per-layer angle lists: the rasterised lines depend on them
    out[name + "_theta_sample"] = {k: [float(x) for x in v.flatten()[:16]] for k, v in m.state_dict().items()
                                   if k.endswith("theta") and ("stages.0.0" in k or "stages.0.1" in k or "dw1" in k)}
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "convnext_keys.json")
json.dump(out, open(path, "w"))
print(path, os.path.getsize(path), {k: v for k, v in out.items() if k.endswith("_params")})
