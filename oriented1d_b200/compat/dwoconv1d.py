"""Bare-name alias: ``from dwoconv1d import DepthwiseOrientedConv1d`` as in the
reference's models/convnext.py:18-20 (general extension)."""
from oriented1d_b200.dwoconv1d import *  # noqa: F401,F403
from oriented1d_b200.dwoconv1d import DepthwiseOrientedConv1d  # noqa: F401
