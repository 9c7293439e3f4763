"""Bare-name alias: ``from dwoconv1d_specialized import DepthwiseOrientedConv1d`` as in
the reference's models/convnext.py:21-23 (per-size specialised extension; here one
prebuilt library serves every size)."""
from oriented1d_b200.dwoconv1d import *  # noqa: F401,F403
from oriented1d_b200.dwoconv1d import DepthwiseOrientedConv1d  # noqa: F401
