"""cgnet_b200: the Clebsch-Gordan layer of CGNet (zlin7/CGNet) as hand-written sm_100a CUDA behind the reference's own
PyTorch module surface.  See include/cgnet_b200.h for the C ABI the modules call."""
from . import cgutils as CGutils  # noqa: F401
from .cg_layers import (CGBN_cuda, CG_woFilter_cuda, MyBatchNormWeightMM_cuda, Plan, get_plan,  # noqa: F401
                        precomputeCG)
from .cgnet import SphericalCNN, SphericalCNN_fast  # noqa: F401
from .s2_sph import SHProjector  # noqa: F401

__version__ = "0.1.0"
