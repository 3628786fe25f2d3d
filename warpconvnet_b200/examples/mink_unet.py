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

import operator
from typing import Optional, Union

import torch
import torch.nn as nn

from ..geometry.types.voxels import Voxels
from ..geometry.coords.search.cache import IntSearchCache
from ..geometry.coords.search.search_results import IntSearchResult
from ..nn.functional.sparse_conv import (STRIDED_CONV_MODE, TILE_ORDER_MIN_OFFSETS, TILE_ORDER_MIN_ROWS, ConvEpilogue,
                                         FusedConvLaunch, FusedRowsLaunch, _identity_map, _implicit_gemm_forward_logic, _merge_bias,
                                         generate_output_coords_and_kernel_map, prefetch_strided_coordinates)
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
        plan = self._launch_plan(x)
        if plan is not None:
            return plan.run(x, restore_order)
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

    def _launch_plan(self, x: Voxels):
        """The network as a list of launch records (:class:`_LaunchPlan`) when it can run that way:
        inference, CUDA, three spatial dimensions, features and every parameter in one of the native
        dtypes.  Rebuilt when a parameter or buffer changes."""
        if self.training or torch.is_grad_enabled() or not isinstance(x, Voxels):
            return None
        feats = x.feature_tensor
        if not feats.is_cuda or x.num_spatial_dims != 3 or feats.dtype != self.final.weight.dtype \
                or feats.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            return None
        plan = self.__dict__.get("_plan")
        if plan is None or not plan.current(feats.dtype, feats.device):
            plan = self.__dict__["_plan"] = _LaunchPlan(self, feats.dtype, feats.device)
        return plan

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


_tensor_version = operator.attrgetter("_version")


class _LaunchPlan:
    """Inference forward of a :class:`MinkUNetBase` as a fixed sequence of
    :class:`FusedConvLaunch` records over per-level neighbour tables.

    The module tree is walked once; per forward only the coordinate work (pyramid, kernel maps)
    and one foreign call per convolution remain, instead of the ``Module`` -> ``Sequential`` ->
    ``spatially_sparse_conv`` stack for each of the 60-odd layers.  The numbers are those of the
    module-by-module path (same kernels, same epilogues, same buffers without concatenation
    copies), and the kernel maps land in the input's shared cache under the same keys."""

    def __init__(self, model: "MinkUNetBase", dtype: torch.dtype, device: torch.device):
        self.dtype, self.device = dtype, device
        self.planes, self.init_dim = model.PLANES, model.INIT_DIM
        self._tensors = list(model.parameters()) + list(model.buffers())
        self._versions = [t._version for t in self._tensors]
        self._ptrs = [t.data_ptr() for t in self._tensors]

        def conv_block(seq, rows_too: bool = False):
            conv, bn = seq[0], seq[1]
            scale, shift = fold_batchnorm(bn)
            ep = _merge_bias(ConvEpilogue(scale=scale, shift=shift), conv.bias)
            relu = isinstance(seq[2], (nn.ReLU, ReLU))
            rec = FusedConvLaunch(conv.weight, dtype, ep.scale, ep.shift, relu=relu)
            if rows_too:  # a 1x1x1 projection: also its input-side record
                return rec, FusedRowsLaunch(conv.weight, dtype, ep.scale, ep.shift, relu=relu)
            return rec

        def basic_block(blk: BasicBlock):
            last = conv_block(blk.conv2)
            last.relu = 1  # relu(conv2 + identity)
            return (conv_block(blk.conv1), last,
                    conv_block(blk.downsample, rows_too=True) if blk.downsample is not None else None)

        def tr_block(blk: ConvTrBlock):
            scale, shift = fold_batchnorm(blk.norm_act[0])
            ep = _merge_bias(ConvEpilogue(scale=scale, shift=shift), blk.conv_tr.bias)
            relu = isinstance(blk.norm_act[1], (nn.ReLU, ReLU))
            return (FusedConvLaunch(blk.conv_tr.weight, dtype, ep.scale, ep.shift, relu=relu),
                    FusedRowsLaunch(blk.conv_tr.weight, dtype, ep.scale, ep.shift, relu=relu))

        assert tuple(model.conv0[0].kernel_size) == (1, 1, 1), "the stem is a 1x1x1 convolution in this plan"
        self.stem = conv_block(model.conv0)
        self.down = [conv_block(m) for m in (model.conv1, model.conv2, model.conv3, model.conv4)]
        self.enc = [[basic_block(b) for b in st] for st in (model.block1, model.block2, model.block3, model.block4)]
        self.up = [tr_block(m) for m in (model.convtr4, model.convtr5, model.convtr6, model.convtr7)]
        self.dec = [[basic_block(b) for b in st] for st in (model.block5, model.block6, model.block7, model.block8)]
        head = model.final
        head_shift = head.bias.detach().float() if head.bias is not None else None
        self.head = FusedConvLaunch(head.weight, dtype, None, head_shift)
        self.head_rows = FusedRowsLaunch(head.weight, dtype, None, head_shift)

    def current(self, dtype, device) -> bool:
        """True while no parameter or buffer has been written or re-allocated since the plan was made
        (version counters and data pointers compared in C loops: this runs on every forward)."""
        if dtype != self.dtype or device != self.device:
            return False
        return (list(map(_tensor_version, self._tensors)) == self._versions
                and list(map(torch.Tensor.data_ptr, self._tensors)) == self._ptrs)

    @staticmethod
    def _blocks(stage, x: torch.Tensor, nbr, rows, n: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        last = len(stage) - 1
        for i, (c1, c2, proj) in enumerate(stage):
            if proj is None:
                identity = x
            elif proj[1].takes(x):   # 1x1x1 projection of the block input: rows streamed once, from the input side
                identity = proj[1](x, None, n)
            else:
                identity = proj[0](x, _identity_map(n, x.device).neighbor_table(n), None, n)
            x = c2(c1(x, nbr, rows, n), nbr, rows, n, residual=identity, out=out if i == last else None)
        return x

    def run(self, x: Voxels, restore_order: bool):
        P, dtype, dev = self.planes, self.dtype, self.device
        ics = [x.batched_coordinates] + prefetch_strided_coordinates(x, [2, 2, 2, 2])
        n = [ic.batched_tensor.shape[0] for ic in ics]
        if x.cache is None:  # one kernel-map cache for the whole forward, as the module path shares it
            x._extra_attributes["_cache"] = IntSearchCache()
        vox = [x] + [x._derive(x.feature_tensor[:0], ic) for ic in ics[1:]]  # coordinate carriers for the map builder
        k3, k2, one = (3, 3, 3), (2, 2, 2), (1, 1, 1)

        def conv3_table(level: int):
            _, _, km = generate_output_coords_and_kernel_map(vox[level], k3, one, one, False, False, None,
                                                             STRIDED_CONV_MODE.STRIDE_ONLY)
            if n[level] >= TILE_ORDER_MIN_ROWS and TILE_ORDER_MIN_OFFSETS <= 27:
                return km.tiled_neighbor_table(n[level])
            return km.neighbor_table(n[level]), None

        def down_table(level: int):  # level -> level + 1
            _, _, km = generate_output_coords_and_kernel_map(vox[level], k2, one, k2, False, False, None,
                                                             STRIDED_CONV_MODE.STRIDE_ONLY)
            return km.neighbor_table(n[level + 1])

        def up_table(level: int):    # level + 1 -> level
            _, _, km = generate_output_coords_and_kernel_map(vox[level + 1], k2, one, k2, False, True, vox[level],
                                                             STRIDED_CONV_MODE.STRIDE_ONLY)
            return km.neighbor_table(n[level])

        def joined(rows: int, c_up: int, c_skip: int):
            buf = torch.empty((rows, c_up + c_skip), dtype=dtype, device=dev)
            return buf, buf[:, :c_up], buf[:, c_up:]

        feats = x.feature_tensor
        if feats.stride(1) != 1:
            feats = feats.contiguous()
        # encoder: every stage writes its result into the right-hand block of its level's skip buffer
        bufs = [joined(n[0], P[7], self.init_dim), joined(n[1], P[6], P[0]), joined(n[2], P[5], P[1]),
                joined(n[3], P[4], P[2])]
        cur = self.stem(feats, _identity_map(n[0], dev).neighbor_table(n[0]), None, n[0], out=bufs[0][2])
        tables = [None] * 5
        children = [None] * 4   # [8, n[level + 1]]: the fine row of every (coarse row, offset), -1 where there is none
        for level in range(4):
            children[level] = down_table(level)
            cur = self.down[level](cur, children[level], None, n[level + 1])
            tables[level + 1] = conv3_table(level + 1)
            nbr, rows = tables[level + 1]
            cur = self._blocks(self.enc[level], cur, nbr, rows, n[level + 1], out=bufs[level + 1][2] if level < 3 else None)
        # decoder: the transposed convolution fills the left-hand block, the stage reads the whole buffer
        for i, level in enumerate((3, 2, 1, 0)):
            buf, left, _ = bufs[level]
            up, up_rows = self.up[i]
            if up_rows.takes(cur):
                # every fine voxel has one parent (the coarse set is the strided fine set): the parents'
                # rows are streamed once and each offset's block written at its child
                up_rows(cur, children[level], n[level], out=left)
            else:
                up(cur, up_table(level), None, n[level], out=left)
            if tables[level] is None:
                tables[level] = conv3_table(level)
            nbr, rows = tables[level]
            cur = self._blocks(self.dec[i], buf, nbr, rows, n[level])
        if restore_order:
            perm = x.extra_attributes.get("perm")
            assert perm is not None, "restore_order needs the permutation that Voxels.sort records"
            # sorted = original[perm], so original row r sits at sorted row inverse[r]: the head reads its
            # input row THROUGH the inverse permutation (whole rows from scattered places) and writes the
            # logits in order, instead of scattering 40-byte rows
            if self.head_rows.takes(cur):
                # sorted row j is original row perm[j]: stream the rows in order, write each at its original place
                dst = perm.to(torch.int32).view(1, n[0]) if perm.dtype != torch.int32 else perm.view(1, n[0])
                return self.head_rows(cur, dst.contiguous(), n[0])
            inverse = torch.empty(n[0], dtype=torch.int32, device=dev)
            inverse[perm] = torch.arange(n[0], dtype=torch.int32, device=dev)
            return self.head(cur, inverse.view(1, n[0]), None, n[0])
        if self.head_rows.takes(cur):
            return x._derive(self.head_rows(cur, None, n[0]))
        return x._derive(self.head(cur, _identity_map(n[0], dev).neighbor_table(n[0]), None, n[0]))


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
