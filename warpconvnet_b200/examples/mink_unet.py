"""MinkUNet family on the sparse-convolution stack, with the layer structure and
parameter names of the reference model (examples/mink_unet.py:25-141, 212-413):
``ConvBlock`` = SparseConv3d(bias=False) -> BatchNorm1d -> ReLU, ``BasicBlock`` =
two 3x3x3 ConvBlocks + (projected) identity + ReLU, ``ConvTrBlock`` = transposed
2x2x2 stride-2 SparseConv3d -> BatchNorm1d -> ReLU, U-shaped encoder/decoder with
skip concatenation and a biased 1x1x1 head.  A reference ``state_dict`` loads
unchanged.  In eval mode every conv -> BN -> (+identity) -> ReLU run executes as
one fused kernel.
"""
from __future__ import annotations

from typing import Optional, Union

import torch
import torch.nn as nn

from ..geometry.types.voxels import Voxels
from ..geometry.coords.search.search_results import IntSearchResult
from ..nn.functional.sparse_conv import ConvEpilogue, _implicit_gemm_forward_logic, prefetch_strided_coordinates
from ..nn.functional.transforms import cat
from ..nn.modules.activations import ReLU
from ..nn.modules.sequential import Sequential, fold_batchnorm
from ..nn.modules.sparse_conv import SparseConv3d


class ConvBlock(Sequential):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1,
                 activation: Optional[nn.Module] = "relu", bias: bool = False,
                 compute_dtype: Optional[torch.dtype] = None):
        act = nn.ReLU(inplace=True) if activation == "relu" else (nn.Identity() if activation is None else activation)
        super().__init__(
            SparseConv3d(in_channels, out_channels, kernel_size, stride, bias=bias, compute_dtype=compute_dtype),
            nn.BatchNorm1d(out_channels),
            act,
        )


class ConvTrBlock(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1,
                 activation: Optional[nn.Module] = "relu", bias: bool = False,
                 compute_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.conv_tr = SparseConv3d(in_channels, out_channels, kernel_size, stride, transposed=True, bias=bias,
                                    compute_dtype=compute_dtype)
        act = nn.ReLU(inplace=True) if activation == "relu" else (nn.Identity() if activation is None else activation)
        self.norm_act = Sequential(nn.BatchNorm1d(out_channels), act)

    def forward(self, x: Voxels, out_spatial_sparsity: Voxels, out: Optional[torch.Tensor] = None) -> Voxels:
        """``out`` (inference only): preallocated destination of the result's features."""
        bn = self.norm_act[0]
        if not bn.training and not (torch.is_grad_enabled() and self.conv_tr.weight.requires_grad):
            scale, shift = fold_batchnorm(bn)
            ep = ConvEpilogue(scale=scale, shift=shift, relu=isinstance(self.norm_act[1], nn.ReLU), out=out)
            return self.conv_tr(x, out_spatial_sparsity, epilogue=ep)
        res = self.norm_act(self.conv_tr(x, out_spatial_sparsity))
        if out is not None:
            out.copy_(res.feature_tensor)
        return res


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_channels: int, out_channels: int, stride: int = 1, bias: bool = False,
                 compute_dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.conv1 = ConvBlock(in_channels, out_channels, kernel_size=3, stride=stride, bias=bias,
                               compute_dtype=compute_dtype)
        self.conv2 = ConvBlock(out_channels, out_channels, kernel_size=3, activation=None, bias=bias,
                               compute_dtype=compute_dtype)
        self.downsample = None
        if stride != 1 or in_channels != out_channels:
            self.downsample = ConvBlock(in_channels, out_channels, kernel_size=1, stride=stride, activation=None,
                                        bias=bias, compute_dtype=compute_dtype)
        self.relu = ReLU(inplace=True)

    def forward(self, x: Voxels, out: Optional[torch.Tensor] = None) -> Voxels:
        """``out`` (inference only): preallocated destination of the block's features."""
        identity = x if self.downsample is None else self.downsample(x)
        y = self.conv1(x)
        # relu(conv2(y) + identity): residual add and ReLU ride in conv2's epilogue
        return self.conv2(y, residual=identity.feature_tensor, final_relu=True, out=out)


class MinkUNetBase(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, planes, layers, init_dim: int = 32,
                 BLOCK: Union[str, nn.Module] = BasicBlock, init_kernel_size: int = 1, **kwargs):
        super().__init__()
        assert len(planes) == len(layers)
        self.PLANES, self.LAYERS, self.INIT_DIM = planes, layers, init_dim
        self.conv0 = ConvBlock(in_channels, init_dim, kernel_size=init_kernel_size, bias=False)
        self.conv1 = ConvBlock(init_dim, init_dim, kernel_size=2, stride=2)
        self.block1 = self._make_layer(BLOCK, init_dim, planes[0], layers[0])
        self.conv2 = ConvBlock(planes[0], planes[0], kernel_size=2, stride=2)
        self.block2 = self._make_layer(BLOCK, planes[0], planes[1], layers[1])
        self.conv3 = ConvBlock(planes[1], planes[1], kernel_size=2, stride=2)
        self.block3 = self._make_layer(BLOCK, planes[1], planes[2], layers[2])
        self.conv4 = ConvBlock(planes[2], planes[2], kernel_size=2, stride=2)
        self.block4 = self._make_layer(BLOCK, planes[2], planes[3], layers[3])
        self.convtr4 = ConvTrBlock(planes[3], planes[4], kernel_size=2, stride=2)
        self.block5 = self._make_layer(BLOCK, planes[4] + planes[2], planes[4], layers[4])
        self.convtr5 = ConvTrBlock(planes[4], planes[5], kernel_size=2, stride=2)
        self.block6 = self._make_layer(BLOCK, planes[5] + planes[1], planes[5], layers[5])
        self.convtr6 = ConvTrBlock(planes[5], planes[6], kernel_size=2, stride=2)
        self.block7 = self._make_layer(BLOCK, planes[6] + planes[0], planes[6], layers[6])
        self.convtr7 = ConvTrBlock(planes[6], planes[7], kernel_size=2, stride=2)
        self.block8 = self._make_layer(BLOCK, planes[7] + planes[0], planes[7], layers[7])
        self.final = SparseConv3d(planes[7], out_channels, kernel_size=1, bias=True)

    @staticmethod
    def _make_layer(BLOCK, in_channels: int, out_channels: int, blocks: int) -> nn.Sequential:
        layers = [BLOCK(in_channels, out_channels)]
        layers += [BLOCK(out_channels, out_channels) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x: Voxels, restore_order: bool = False):
        """``restore_order`` (an addition to the reference signature; inference only): ``x`` is the
        result of ``Voxels.sort`` and the logits are wanted for the rows as they were before the
        sort.  The last convolution then stores its rows through the sort permutation and the
        return value is the ``[N, classes]`` tensor in that order, with no separate un-permute."""
        # all four coarse coordinate sets first: their size read-backs then wait for coordinate
        # kernels only, and the convolutions below queue without a host synchronisation
        prefetch_strided_coordinates(x, [2, 2, 2, 2])
        if self.training or torch.is_grad_enabled():
            out_p1 = self.conv0(x)
            out_b1p2 = self.block1(self.conv1(out_p1))
            out_b2p4 = self.block2(self.conv2(out_b1p2))
            out_b3p8 = self.block3(self.conv3(out_b2p4))
            out = self.block4(self.conv4(out_b3p8))
            out = self.block5(cat(self.convtr4(out, out_b3p8), out_b3p8))
            out = self.block6(cat(self.convtr5(out, out_b2p4), out_b2p4))
            out = self.block7(cat(self.convtr6(out, out_b1p2), out_b1p2))
            out = self.block8(cat(self.convtr7(out, out_p1), out_p1))
        else:
            out = self._forward_joined(x)
        if restore_order:
            perm = x.extra_attributes.get("perm")
            assert perm is not None, "restore_order needs the permutation that Voxels.sort records"
            # sorted = original[perm], so original row r sits at sorted row inverse[r]: the head reads its
            # input row THROUGH the inverse permutation (whole 192-byte rows from scattered places) and
            # writes the logits in order, instead of scattering 40-byte rows
            n = perm.shape[0]
            inverse = torch.empty(n, dtype=torch.int32, device=perm.device)
            inverse[perm] = torch.arange(n, dtype=torch.int32, device=perm.device)
            unsort = IntSearchResult.from_neighbor_table(inverse.view(1, n), n, None, None)
            bias = self.final.bias
            ep = ConvEpilogue(shift=bias.detach().float()) if bias is not None else None
            return _implicit_gemm_forward_logic(out.feature_tensor, self.final.weight, unsort, n, None, epilogue=ep)
        return self.final(out)

    def _forward_joined(self, x: Voxels) -> Voxels:
        """Inference body without concatenation copies.  Each skip connection ``cat(up, skip)`` is
        one buffer ``[M, C_up + C_skip]`` allocated when the encoder reaches that level: the encoder
        stage writes its result straight into the right-hand column block (and the next stage reads
        it from there, rows ``C_up + C_skip`` elements apart), the transposed convolution of the
        decoder later fills the left-hand block, and the decoder stage reads the whole buffer."""
        P = self.PLANES
        dtype, dev = x.feature_tensor.dtype, x.feature_tensor.device

        def joined(rows: int, c_up: int, c_skip: int):
            buf = torch.empty((rows, c_up + c_skip), dtype=dtype, device=dev)
            return buf, buf[:, :c_up], buf[:, c_up:]

        def stage(blocks: nn.Sequential, v: Voxels, out: torch.Tensor) -> Voxels:
            n = len(blocks)
            for i, blk in enumerate(blocks):
                v = blk(v, out=out if i == n - 1 else None)
            return v

        buf8, up8, skip8 = joined(len(x), P[7], self.INIT_DIM)
        out_p1 = self.conv0(x, out=skip8)
        v = self.conv1(out_p1)
        buf7, up7, skip7 = joined(len(v), P[6], P[0])
        out_b1p2 = stage(self.block1, v, skip7)
        v = self.conv2(out_b1p2)
        buf6, up6, skip6 = joined(len(v), P[5], P[1])
        out_b2p4 = stage(self.block2, v, skip6)
        v = self.conv3(out_b2p4)
        buf5, up5, skip5 = joined(len(v), P[4], P[2])
        out_b3p8 = stage(self.block3, v, skip5)
        v = self.block4(self.conv4(out_b3p8))
        self.convtr4(v, out_b3p8, out=up5)
        v = self.block5(out_b3p8._derive(buf5))
        self.convtr5(v, out_b2p4, out=up6)
        v = self.block6(out_b2p4._derive(buf6))
        self.convtr6(v, out_b1p2, out=up7)
        v = self.block7(out_b1p2._derive(buf7))
        self.convtr7(v, out_p1, out=up8)
        return self.block8(out_p1._derive(buf8))


class MinkUNet18(MinkUNetBase):
    def __init__(self, in_channels: int, out_channels: int, **kwargs):
        super().__init__(in_channels, out_channels, planes=(32, 64, 128, 256, 256, 128, 96, 96),
                         layers=(2, 2, 2, 2, 2, 2, 2, 2), init_dim=32, BLOCK=BasicBlock, **kwargs)


class MinkUNet34(MinkUNetBase):
    def __init__(self, in_channels: int, out_channels: int, **kwargs):
        super().__init__(in_channels, out_channels, planes=(32, 64, 128, 256, 256, 128, 96, 96),
                         layers=(2, 3, 4, 6, 2, 2, 2, 2), init_dim=32, BLOCK=BasicBlock, **kwargs)


@torch.no_grad()
def randomize_batchnorm_(model: nn.Module, seed: int = 0) -> None:
    """Seeded, non-trivial BatchNorm parameters and running statistics, so that an
    eval-mode comparison exercises the folded scale/shift instead of an identity."""
    g = torch.Generator().manual_seed(seed)
    for m in model.modules():
        if isinstance(m, nn.BatchNorm1d):
            c = m.num_features
            m.weight.copy_(torch.rand(c, generator=g) + 0.5)
            m.bias.copy_(torch.randn(c, generator=g) * 0.1)
            m.running_mean.copy_(torch.randn(c, generator=g) * 0.1)
            m.running_var.copy_(torch.rand(c, generator=g) * 0.5 + 0.75)
