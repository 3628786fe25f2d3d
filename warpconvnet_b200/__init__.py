"""B200-native sparse convolution behind the WarpConvNet surface.

Geometry: :class:`Voxels`, :class:`IntCoords`, :class:`CatFeatures`;
search: :class:`TorchHashTable`, :func:`generate_kernel_map`, :class:`IntSearchResult`;
layers: :class:`SparseConv3d`, :func:`spatially_sparse_conv`, :class:`Sequential`.
All compute runs in ``csrc/libwcn_b200.so`` (hand-written sm_100a CUDA behind a C
ABI, ``include/wcn_b200.h``); there is no CPU path.
"""
from .geometry.coords.integer import IntCoords
from .geometry.coords.ops.serialization import POINT_ORDERING, encode, morton_code
from .geometry.coords.ops.stride import stride_coords
from .geometry.coords.search.cache import IntSearchCache, IntSearchCacheKey
from .geometry.coords.search.search_results import IntSearchResult
from .geometry.coords.search.torch_discrete import generate_kernel_map, kernel_offsets_from_size
from .geometry.coords.search.torch_hashmap import HashMethod, TorchHashTable
from .geometry.features.cat import CatFeatures
from .geometry.types.voxels import Voxels
from .nn.functional.sparse_conv import (SPARSE_CONV_BWD_ALGO_MODE, SPARSE_CONV_FWD_ALGO_MODE, STRIDED_CONV_MODE,
                                        ConvEpilogue, spatially_sparse_conv)
from .nn.functional.sparse_pool import sparse_avg_pool, sparse_max_pool, sparse_reduce, sparse_unpool
from .nn.functional.transforms import cat
from .nn.modules.activations import ReLU
from .nn.modules.normalizations import BatchNorm
from .nn.modules.sequential import Sequential
from .nn.modules.sparse_conv import SparseConv2d, SparseConv3d, SpatiallySparseConv
from .nn.modules.sparse_pool import SparseMaxPool, SparseMinPool, SparsePool, SparseUnpool
from .ops.reductions import REDUCTIONS

__version__ = "0.1.0"
