"""Layer front ends: the parts of ``torkit3d.layers.pointnet2`` that sit on the operators."""
from .pointnet2 import (BallQuery, FeatureInterpolator, SetAbstractionGrouper, sample_and_gather,
                        set_abstraction_group, three_nn_interpolate)

__all__ = ["BallQuery", "FeatureInterpolator", "SetAbstractionGrouper", "sample_and_gather",
           "set_abstraction_group", "three_nn_interpolate"]
