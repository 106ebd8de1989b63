"""cusync_b200 -- B200-native CuSync: tile-level synchronisation of dependent
GPU kernels, with hand-written sm_100a GEMM kernels behind the reference's
CuStage / CuSync / policy API.  Python here is a thin host-side mirror of that
API over the library's C ABI."""
from . import _lib
from ._lib import CuSyncError, CuSyncLibraryError  # noqa: F401
from .api import (CuStage, CuSync, NoSync, RowSync, TileSync, StridedTileSync, Conv2DTileSync,  # noqa: F401
                  ConsecutiveTileSync, IdentityOrder, TransposeXYOrder, GroupedRowsOrder, Optimizations, Gemm, GemmArguments,
                  gemm_tiled_shape, Conv2dFprop, Conv2dProblemSize)
from .mlp import MLPShard, make_inputs  # noqa: F401,E402
from .conv import ConvChain  # noqa: F401,E402
