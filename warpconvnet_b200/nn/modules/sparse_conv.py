"""Sparse-convolution modules (warpconvnet/nn/modules/sparse_conv.py:30-374).

Parameters keep the reference's names, shapes and initialisation — ``weight
[K, C_in, C_out]``, optional ``bias [C_out]`` — so its ``state_dict`` loads as is.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import numpy as np
import torch
import torch.nn as nn
from torch.nn.init import calculate_gain

from ...constants import WARPCONVNET_BWD_ALGO_MODE, WARPCONVNET_FWD_ALGO_MODE
from ...geometry.coords.ops.serialization import POINT_ORDERING
from ...geometry.types.voxels import Voxels
from ...utils.ntuple import ntuple
from ..functional.sparse_conv import (SPARSE_CONV_BWD_ALGO_MODE, SPARSE_CONV_FWD_ALGO_MODE, STRIDED_CONV_MODE,
                                      ConvEpilogue, spatially_sparse_conv)
from .base_module import BaseSpatialModule


class SpatiallySparseConv(BaseSpatialModule):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: Union[int, Tuple[int, ...]],
                 stride: Union[int, Tuple[int, ...]] = 1, dilation: Union[int, Tuple[int, ...]] = 1,
                 bias: bool = True, transposed: bool = False, generative: bool = False,
                 kernel_matmul_batch_size: int = 2, num_spatial_dims: Optional[int] = 3,
                 fwd_algo: Optional[Union[SPARSE_CONV_FWD_ALGO_MODE, str]] = None,
                 bwd_algo: Optional[Union[SPARSE_CONV_BWD_ALGO_MODE, str]] = None,
                 stride_mode: STRIDED_CONV_MODE = STRIDED_CONV_MODE.STRIDE_ONLY,
                 order: POINT_ORDERING = POINT_ORDERING.RANDOM, compute_dtype: Optional[torch.dtype] = None,
                 implicit_matmul_fwd_block_size: Optional[int] = None,
                 implicit_matmul_bwd_block_size: Optional[int] = None):
        super().__init__()
        self.num_spatial_dims = num_spatial_dims
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = ntuple(kernel_size, ndim=num_spatial_dims)
        self.stride = ntuple(stride, ndim=num_spatial_dims)
        self.dilation = ntuple(dilation, ndim=num_spatial_dims)
        self.transposed, self.generative = transposed, generative
        self.kernel_matmul_batch_size = kernel_matmul_batch_size
        # constructor argument, else the environment default (reference :110-126)
        fwd_algo = WARPCONVNET_FWD_ALGO_MODE if fwd_algo is None else fwd_algo
        bwd_algo = WARPCONVNET_BWD_ALGO_MODE if bwd_algo is None else bwd_algo
        self.fwd_algo = SPARSE_CONV_FWD_ALGO_MODE(fwd_algo) if isinstance(fwd_algo, str) else fwd_algo
        self.bwd_algo = SPARSE_CONV_BWD_ALGO_MODE(bwd_algo) if isinstance(bwd_algo, str) else bwd_algo
        self.stride_mode, self.order, self.compute_dtype = stride_mode, order, compute_dtype
        self.implicit_matmul_fwd_block_size = implicit_matmul_fwd_block_size
        self.implicit_matmul_bwd_block_size = implicit_matmul_bwd_block_size
        self.weight = nn.Parameter(torch.empty(int(np.prod(self.kernel_size)), in_channels, out_channels))
        self.bias = nn.Parameter(torch.empty(out_channels)) if bias else None
        self.reset_parameters()

    def __repr__(self):
        s = (f"{self.__class__.__name__}(in_channels={self.in_channels}, out_channels={self.out_channels}, "
             f"kernel_size={self.kernel_size}")
        if any(v != 1 for v in self.stride):
            s += f", stride={self.stride}"
        if any(v != 1 for v in self.dilation):
            s += f", dilation={self.dilation}"
        if self.transposed:
            s += f", transposed={self.transposed}"
        if self.generative:
            s += f", generative={self.generative}"
        if self.order != POINT_ORDERING.RANDOM:
            s += f", order={self.order}"
        return s + ")"

    def _calculate_fan_in_and_fan_out(self):
        rf = int(np.prod(self.kernel_size))
        return self.in_channels * rf, self.out_channels * rf

    @torch.no_grad()
    def reset_parameters(self):
        """uniform(+-sqrt(D) * gain(leaky_relu, sqrt 5) / sqrt(fan)), fan_in (fan_out when
        transposed); bias uniform(+-1/sqrt(fan_in)) (reference :159-191)."""
        fan_in, fan_out = self._calculate_fan_in_and_fan_out()
        fan = fan_out if self.transposed else fan_in
        std = calculate_gain("leaky_relu", math.sqrt(5)) / math.sqrt(fan)
        bound = math.sqrt(self.num_spatial_dims) * std
        self.weight.uniform_(-bound, bound)
        if self.bias is not None:
            b = 1 / math.sqrt(fan_in)
            self.bias.uniform_(-b, b)

    def forward(self, input_sparse_tensor: Voxels, output_spatially_sparse_tensor: Optional[Voxels] = None,
                epilogue: Optional[ConvEpilogue] = None):
        return spatially_sparse_conv(
            input_sparse_tensor=input_sparse_tensor, weight=self.weight, kernel_size=self.kernel_size,
            stride=self.stride, kernel_dilation=self.dilation, bias=self.bias,
            kernel_matmul_batch_size=self.kernel_matmul_batch_size,
            output_spatially_sparse_tensor=output_spatially_sparse_tensor, transposed=self.transposed,
            generative=self.generative, fwd_algo=self.fwd_algo, bwd_algo=self.bwd_algo,
            stride_mode=self.stride_mode, order=self.order, compute_dtype=self.compute_dtype,
            implicit_matmul_fwd_block_size=self.implicit_matmul_fwd_block_size,
            implicit_matmul_bwd_block_size=self.implicit_matmul_bwd_block_size, epilogue=epilogue)


class SparseConv2d(SpatiallySparseConv):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, dilation=1, bias=True, transposed=False,
                 generative: bool = False, stride_mode: STRIDED_CONV_MODE = STRIDED_CONV_MODE.STRIDE_ONLY,
                 fwd_algo=None, bwd_algo=None, kernel_matmul_batch_size: int = 2,
                 order: POINT_ORDERING = POINT_ORDERING.RANDOM, compute_dtype: Optional[torch.dtype] = None,
                 implicit_matmul_fwd_block_size: Optional[int] = None,
                 implicit_matmul_bwd_block_size: Optional[int] = None):
        super().__init__(in_channels, out_channels, kernel_size, stride, dilation, bias, transposed, generative,
                         kernel_matmul_batch_size, 2, fwd_algo, bwd_algo, stride_mode, order, compute_dtype,
                         implicit_matmul_fwd_block_size, implicit_matmul_bwd_block_size)


class SparseConv3d(SpatiallySparseConv):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, dilation=1, bias=True, transposed=False,
                 generative: bool = False, stride_mode: STRIDED_CONV_MODE = STRIDED_CONV_MODE.STRIDE_ONLY,
                 fwd_algo=None, bwd_algo=None, kernel_matmul_batch_size: int = 2,
                 order: POINT_ORDERING = POINT_ORDERING.RANDOM, compute_dtype: Optional[torch.dtype] = None,
                 implicit_matmul_fwd_block_size: Optional[int] = None,
                 implicit_matmul_bwd_block_size: Optional[int] = None):
        super().__init__(in_channels, out_channels, kernel_size, stride, dilation, bias, transposed, generative,
                         kernel_matmul_batch_size, 3, fwd_algo, bwd_algo, stride_mode, order, compute_dtype,
                         implicit_matmul_fwd_block_size, implicit_matmul_bwd_block_size)
