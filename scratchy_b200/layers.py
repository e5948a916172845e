"""Host-side mirror of the reference's quantized-linear layer and loader interface.

Reference (paths relative to its root):
  * payload types        crates/models/quantization/src/layers_quant.rs:33-52 (`AffineQuantLinear`),
                         crates/layers/src/layers.rs:179-191 (`Fp8Linear`), :212-236 (`LinearLayer`)
  * loaders              crates/targets/metal/src/layers_quant.rs:289-345 (`MetalAffineQuantOps::load`),
                         crates/targets/metal/src/loaders.rs:96-116 (`load_layered_linear_affine_quant`)
  * weight store         crates/layers/src/weights.rs (`GpuWeights::take`, `contains`)
  * the forward step     crates/targets/metal/src/tape/step.rs:456-470 (`AffineMatmul`)

Names, argument meaning and error behaviour follow those; the arithmetic runs only in the
CUDA library (``_lib``).  torch tensors are used as device buffers and for the stream.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import _lib
from ._lib import KIND_AFFINE_B4, KIND_FP8_DYNAMIC, ScratchyCudaError


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dev_index(device) -> int:
    d = torch.device(device)
    return d.index if d.index is not None else torch.cuda.current_device()


class GpuWeights:
    """A named store of device tensors, the loader vocabulary of `GpuWeights` in the reference
    (crates/layers/src/weights.rs): `take` removes and returns a tensor, `contains` probes."""

    def __init__(self, tensors: Dict[str, torch.Tensor], scale_dtype: Optional[torch.dtype] = torch.bfloat16):
        self._t = dict(tensors)
        self._scale_dtype = scale_dtype

    def contains(self, name: str) -> bool:
        return name in self._t

    def take(self, name: str) -> torch.Tensor:
        if name not in self._t:
            raise KeyError(f"tensor `{name}` not found in checkpoint")
        return self._t.pop(name)

    def peek(self, name: str) -> torch.Tensor:
        """The tensor without removing it (`copy_cpu` in the reference leaves the part in the store)."""
        if name not in self._t:
            raise KeyError(f"tensor `{name}` not found in checkpoint")
        return self._t[name]

    def rmsnorm_scale_dtype(self) -> Optional[torch.dtype]:
        return self._scale_dtype


def affine_packed_cols(in_features: int, bits: int) -> int:
    """crates/targets/metal/src/layers_quant.rs:46-48."""
    return (in_features * bits + 31) // 32


@dataclass
class AffineQuantLinear:
    """MLX affine int4 linear, repacked for the B200 kernels at load time.

    `packed` is the streaming layout written by `scr_affine_b4_repack`; the checkpoint
    tensors are released after the repack unless `keep_source` was set.
    """
    packed: torch.Tensor
    in_features: int
    out_features: int
    group_size: int
    bits: int
    linear_bias: Optional[torch.Tensor] = None
    source: Optional[dict] = field(default=None, repr=False)
    pairs8: bool = False        # rows interleaved 8 gate / 8 up (see `load_rows_interleave8`)

    # ---- MetalAffineQuantOps::load (layers_quant.rs:289-345)
    @classmethod
    def load(cls, weights: GpuWeights, prefix: str, group_size: int, bits: int, expected_in_features: int,
             keep_source: bool = False) -> "AffineQuantLinear":
        weight = weights.take(f"{prefix}.weight")
        scales = _take_affine_scales(weights, f"{prefix}.scales")
        affine_biases = _take_affine_scales(weights, f"{prefix}.biases")
        linear_bias = weights.take(f"{prefix}.bias") if weights.contains(f"{prefix}.bias") else None
        if weight.dim() != 2:
            raise ValueError(f"`{prefix}.weight` must be 2-D, got {tuple(weight.shape)}")
        out_features, packed_cols = int(weight.shape[0]), int(weight.shape[1])
        in_features = packed_cols * 32 // bits
        if (packed_cols * 32) % bits != 0 or affine_packed_cols(in_features, bits) != packed_cols:
            raise ValueError(
                f"affine quant checkpoint/preset mismatch at `{prefix}`: packed `.weight` is "
                f"[{out_features}, {packed_cols}], implying in_features={in_features} at bits={bits}; "
                f"this build expects in_features={expected_in_features}.")
        if in_features != expected_in_features:
            raise ValueError(
                f"affine quant checkpoint/preset mismatch at `{prefix}`: packed `.weight` implies "
                f"in_features={in_features} at bits={bits}, but this build expects "
                f"in_features={expected_in_features}")
        if in_features % group_size != 0:
            raise ValueError(f"`{prefix}`: in_features={in_features} not divisible by group_size={group_size}")
        want = (out_features, in_features // group_size)
        if tuple(scales.shape) != want or tuple(affine_biases.shape) != want:
            raise ValueError(f"`{prefix}`: scales/biases must be {want}, got {tuple(scales.shape)} / "
                             f"{tuple(affine_biases.shape)}")
        return cls.from_tensors(weight, scales, affine_biases, group_size, bits, linear_bias, keep_source)

    # ---- MetalAffineQuantOps::load_rows_concat (layers_quant.rs:363-450): fused QKV / gate-up
    @staticmethod
    def _collect_parts(weights: GpuWeights, prefixes, group_size: int, bits: int, expected_in_features: int):
        """The checks of `load_rows_concat` (layers_quant.rs:363-430); returns the parts' codes, scales, biases."""
        if not prefixes:
            raise ValueError("AffineQuantLinear::load_rows_concat: empty prefix list")
        compiled = weights.rmsnorm_scale_dtype()
        if compiled is None:
            raise ValueError(f"`{prefixes[0]}.scales`: no scale dtype pinned")
        codes, scales, biases = [], [], []
        widths = None
        for prefix in prefixes:
            if weights.contains(f"{prefix}.bias"):
                raise ValueError(f"affine rows concat: `{prefix}.bias` present — a fused projection carries no bias")
            w, sc, b = weights.peek(f"{prefix}.weight"), weights.peek(f"{prefix}.scales"), weights.peek(f"{prefix}.biases")
            if w.dtype not in (torch.int32, torch.uint32) or w.dim() != 2:
                raise ValueError(f"affine rows concat: `{prefix}.weight` is {w.dtype} {tuple(w.shape)} "
                                 "(expected U32 rank 2)")
            for name, t in (("scales", sc), ("biases", b)):
                if t.dtype != compiled:
                    raise ValueError(f"`{prefix}.{name}` is {t.dtype} on disk; this build's quantized kernels "
                                     f"read {compiled}")
            rows, packed_cols = int(w.shape[0]), int(w.shape[1])
            in_features = packed_cols * 32 // bits
            if affine_packed_cols(in_features, bits) != packed_cols or in_features != expected_in_features:
                raise ValueError(f"affine rows concat: `{prefix}.weight` [{rows}, {packed_cols}] is not a bits={bits} "
                                 f"packing of in_features={expected_in_features}")
            groups = in_features // group_size
            if tuple(sc.shape) != (rows, groups) or tuple(b.shape) != (rows, groups):
                raise ValueError(f"affine rows concat: `{prefix}` scales {tuple(sc.shape)} / biases "
                                 f"{tuple(b.shape)} are not [{rows}, {groups}]")
            if widths is None:
                widths = (packed_cols, groups)
            elif widths != (packed_cols, groups):
                raise ValueError(f"affine rows concat: `{prefix}` row width differs from the first part's")
            codes.append(w)
            scales.append(sc)
            biases.append(b)
        return codes, scales, biases

    # ---- MetalAffineQuantOps::load_rows_concat (layers_quant.rs:363-450): fused QKV / gate-up
    @classmethod
    def load_rows_concat(cls, weights: GpuWeights, prefixes, group_size: int, bits: int,
                         expected_in_features: int) -> "AffineQuantLinear":
        """One projection made of several projections' rows, in order.  A group runs along K, so a
        row dequantises from its own codes, scale and bias wherever it sits.  A part's linear bias
        is refused, not dropped; the parts stay in the store."""
        codes, scales, biases = cls._collect_parts(weights, prefixes, group_size, bits, expected_in_features)
        return cls.from_tensors(torch.cat(codes, 0), torch.cat(scales, 0), torch.cat(biases, 0), group_size, bits)

    @classmethod
    def load_rows_interleave8(cls, weights: GpuWeights, gate_prefix: str, up_prefix: str, group_size: int, bits: int,
                              expected_in_features: int) -> "AffineQuantLinear":
        """The fused gate/up projection in the row order of the fused silu*up epilogue: per 16 rows, 8 gate
        rows then the 8 up rows of the same channels.  Same checks as `load_rows_concat`."""
        (w, wu), (sc, su), (b, bu) = cls._collect_parts(weights, [gate_prefix, up_prefix], group_size, bits,
                                                        expected_in_features)
        inter = int(w.shape[0])
        if w.shape[0] != wu.shape[0]:
            raise ValueError("gate/up interleave: the two projections differ in out_features")
        if inter % 8:
            raise ValueError(f"gate/up interleave: {inter} channels per projection is not a multiple of 8")

        def weave(a, c):
            return torch.stack([a.reshape(inter // 8, 8, -1), c.reshape(inter // 8, 8, -1)], dim=1).reshape(2 * inter, -1)
        out = cls.from_tensors(weave(w, wu), weave(sc, su), weave(b, bu), group_size, bits)
        out.pairs8 = True
        return out

    def forward_silu_mul(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                         scratch: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`silu(x @ gate^T) * (x @ up^T)` on a matrix built by `load_rows_interleave8`: one launch up to 16
        tokens (`scr_linear_affine_b4_silu_mul`), the linear into `scratch` plus `scr_silu_mul_pairs8_bf16` above."""
        if not getattr(self, "pairs8", False):
            raise ValueError("forward_silu_mul needs a gate/up matrix built by load_rows_interleave8")
        if self.linear_bias is not None:
            raise ValueError("the fused silu*up epilogue has no bias end: a `.bias` on gate/up is refused, not dropped")
        x2 = x.reshape(-1, self.in_features).contiguous()
        M, inter = int(x2.shape[0]), self.out_features // 2
        dev = x2.device
        if out is None:
            out = torch.empty((M, inter), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        if M <= 16:
            ctx.check(_lib.lib().scr_linear_affine_b4_silu_mul(ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features,
                                                               self.in_features, self.group_size, _ptr(out), _stream(dev)))
            return out
        if scratch is None:
            scratch = torch.empty((M, self.out_features), dtype=torch.bfloat16, device=dev)
        self.forward(x2, out=scratch, workspace=workspace)
        ctx.check(_lib.lib().scr_silu_mul_pairs8_bf16(ctx.handle, _ptr(scratch), int(scratch.stride(0)), _ptr(out), M, inter,
                                                      _stream(dev)))
        return out

    @classmethod
    def from_tensors(cls, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
                     bits: int = 4, linear_bias: Optional[torch.Tensor] = None,
                     keep_source: bool = False) -> "AffineQuantLinear":
        if bits != 4:
            raise ScratchyCudaError(-4, f"bits={bits}: the cuda target implements the 4-bit preset only")
        if weight.dtype not in (torch.int32, torch.uint32):
            raise ValueError(f"`.weight` must be U32, got {weight.dtype}")
        if scales.dtype not in (torch.bfloat16, torch.float16) or biases.dtype != scales.dtype:
            raise ValueError(f"scales/biases must both be F16 or both BF16, got {scales.dtype} / {biases.dtype}")
        scale_dtype = _lib.DTYPE_F16 if scales.dtype == torch.float16 else _lib.DTYPE_BF16
        if not weight.is_cuda:
            raise ScratchyCudaError(-5, "weights must be on a CUDA device (there is no CPU path)")
        dev = weight.device
        N, K = int(weight.shape[0]), int(weight.shape[1]) * 8
        if linear_bias is not None:
            # `{prefix}.bias` (layers_quant.rs:318-351): one value per output channel, in the activation dtype
            if linear_bias.dtype != torch.bfloat16 or tuple(linear_bias.shape) != (N,):
                raise ValueError(f"`.bias` must be bf16 [{N}], got {linear_bias.dtype} {tuple(linear_bias.shape)}")
            linear_bias = linear_bias.to(dev).contiguous()
        ctx = _lib.context(_dev_index(dev))
        L = _lib.lib()
        size = ctypes.c_size_t(0)
        ctx.check(L.scr_affine_b4_repack_size(N, K, group_size, ctypes.byref(size)))
        packed = torch.empty(size.value, dtype=torch.uint8, device=dev)
        weight, scales, biases = weight.contiguous(), scales.contiguous(), biases.contiguous()
        ctx.check(L.scr_affine_b4_repack(ctx.handle, _ptr(weight), _ptr(scales), _ptr(biases), scale_dtype, N, K, group_size,
                                         _ptr(packed), _stream(dev)))
        src = {"weight": weight, "scales": scales, "biases": biases} if keep_source else None
        return cls(packed, K, N, group_size, bits, linear_bias, src)

    def workspace_bytes(self, M: int) -> int:
        size = ctypes.c_size_t(0)
        st = _lib.lib().scr_linear_workspace_size(KIND_AFFINE_B4, M, self.out_features, self.in_features,
                                                  ctypes.byref(size))
        if st:
            raise ScratchyCudaError(st, "scr_linear_workspace_size")
        return size.value

    # ---- the `AffineMatmul` step (tape/step.rs:456-470): y = x @ dequant(W)^T
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("x must be a bf16 CUDA tensor")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"x has {x.shape[-1]} features, layer expects {self.in_features}")
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if out is None:
            out = torch.empty((M, self.out_features), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        need = self.workspace_bytes(M)
        if need and (workspace is None or workspace.numel() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ctx.check(_lib.lib().scr_linear_affine_b4(
            ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features, self.in_features, self.group_size,
            _ptr(self.linear_bias), _ptr(out), _ptr(workspace), ctypes.c_size_t(workspace.numel() if workspace is not None else 0),
            _stream(dev)))
        return out.reshape(*x.shape[:-1], self.out_features)

    @staticmethod
    def forward_group(layers, x: torch.Tensor, outs=None, workspace: Optional[torch.Tensor] = None):
        """Up to 4 linears over the SAME activations (q, k, v; gate, up) as one launch (`scr_linear_affine_b4_group`): each
        keeps its own packed buffer and gets its own output, the bits of `forward` per member.  Returns the outputs."""
        layers = list(layers)
        if not 1 <= len(layers) <= 4:
            raise ValueError(f"a group holds 1 to 4 linears, got {len(layers)}")
        K, g = layers[0].in_features, layers[0].group_size
        if any(l.in_features != K or l.group_size != g for l in layers):
            raise ValueError("the linears of a group share in_features and the group size")
        if any(l.linear_bias is not None for l in layers):
            raise ValueError("a group launch has no bias end: a `.bias` is refused, not dropped")
        x2 = x.reshape(-1, K).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if outs is None:
            outs = [torch.empty((M, l.out_features), dtype=torch.bfloat16, device=dev) for l in layers]
        n = len(layers)
        packed = (ctypes.c_void_p * n)(*[l.packed.data_ptr() for l in layers])
        ys = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
        ns = (ctypes.c_int32 * n)(*[l.out_features for l in layers])
        ws_ptr, ws_bytes = (_ptr(workspace), workspace.numel() * workspace.element_size()) if workspace is not None else (None, 0)
        if M > 16 and workspace is None:
            need = max(l.workspace_bytes(M) for l in layers)
            if need:
                workspace = torch.empty(need, dtype=torch.uint8, device=dev)
                ws_ptr, ws_bytes = _ptr(workspace), need
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_linear_affine_b4_group(ctx.handle, n, packed, _ptr(x2), M, ns, K, g, ys, ws_ptr,
                                                        ctypes.c_size_t(ws_bytes), _stream(dev)))
        return outs

    def forward_ends(self, x: torch.Tensor, out: torch.Tensor, norm_gain: Optional[torch.Tensor] = None, norm_eps: float = 0.0,
                     norm_gain_offset: float = 0.0, scale: float = 1.0, residual: bool = False, silu_pairs: bool = False,
                     norm_row_scale: bool = False) -> torch.Tensor:
        """The matvec with the reference's `QmvEnds` around it (`scr_linear_affine_b4_ends`, up to 16 tokens): RMSNorm on the
        input as it is loaded (`norm_gain`: x is the norm's INPUT), the layer's bias, a scale, and either the add into the
        residual stream `out` (`residual`) or the gate/up pairing (`silu_pairs`, a matrix built by `load_rows_interleave8`).
        `norm_row_scale`: the reference matvec's own norm-in arithmetic (dot over `x * gain`, the row scaled by `1 / rms(x)`;
        crates/targets/metal/tests/affine_qmv_ends_test.rs:6-9) instead of the bits of the separate RMSNorm."""
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if silu_pairs and not getattr(self, "pairs8", False):
            raise ValueError("silu_pairs needs a gate/up matrix built by load_rows_interleave8")
        ends = _lib.QmvEnds(_ptr(norm_gain), float(norm_eps), float(norm_gain_offset), _ptr(self.linear_bias), float(scale),
                            int(residual), int(silu_pairs), int(norm_row_scale))
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_linear_affine_b4_ends(ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features, self.in_features,
                                                       self.group_size, ctypes.byref(ends), _ptr(out), _stream(dev)))
        return out

    @staticmethod
    def norm_in_supported(M: int, K: int) -> bool:
        """Whether the norm-in end takes M rows of K features (the normalised rows sit in shared memory)."""
        return M <= 8 and M * K * 2 <= 20 * 1024

    ENDS_SCRATCH_BYTES = 65536      # SCR_ENDS_SCRATCH_BYTES

    def forward_residual_rmsnorm(self, x: torch.Tensor, residual: torch.Tensor, gain: torch.Tensor, eps: float,
                                 normed: torch.Tensor, scratch: torch.Tensor,
                                 delta: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`residual += x @ W^T` (in place, bf16) and `normed = rmsnorm(residual, gain)`: one launch up to 16 tokens
        (`scr_linear_affine_b4_residual_rmsnorm`; `scratch` = ENDS_SCRATCH_BYTES, zeroed once by the caller), the
        linear into `delta` followed by `scr_fused_add_rmsnorm_bf16` above."""
        if self.linear_bias is not None:
            raise ValueError("the fused residual + norm epilogue has no bias end: a `.bias` is refused, not dropped")
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        ctx = _lib.context(_dev_index(dev))
        if M <= 16:
            ctx.check(_lib.lib().scr_linear_affine_b4_residual_rmsnorm(
                ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features, self.in_features, self.group_size,
                _ptr(residual), _ptr(gain), ctypes.c_float(eps), _ptr(normed), _ptr(scratch),
                ctypes.c_size_t(scratch.numel() * scratch.element_size()), _stream(dev)))
            return normed
        delta = self.forward(x2, out=delta, workspace=workspace)
        ctx.check(_lib.lib().scr_fused_add_rmsnorm_bf16(ctx.handle, _ptr(residual), _ptr(delta), _ptr(gain), _ptr(normed), M,
                                                        self.out_features, ctypes.c_float(eps), _stream(dev)))
        return normed

    def forward_partial(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                        workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel use: unrounded f32 sums over this rank's K-slice (`scr_linear_affine_b4_partial`)."""
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if out is None:
            out = torch.empty((M, self.out_features), dtype=torch.float32, device=dev)
        ctx = _lib.context(_dev_index(dev))
        need = self.workspace_bytes(M)
        if need and (workspace is None or workspace.numel() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ctx.check(_lib.lib().scr_linear_affine_b4_partial(
            ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features, self.in_features, self.group_size,
            _ptr(out), _ptr(workspace), ctypes.c_size_t(workspace.numel() if workspace is not None else 0),
            _stream(dev)))
        return out

    def dequantize(self) -> torch.Tensor:
        """Test hook: dense bf16 [N, K] from the repacked buffer (`scr_affine_b4_dequant_dump`)."""
        dev = self.packed.device
        w = torch.empty((self.out_features, self.in_features), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_affine_b4_dequant_dump(ctx.handle, _ptr(self.packed), self.out_features,
                                                        self.in_features, self.group_size, _ptr(w), _stream(dev)))
        return w


@dataclass
class AffineQuantEmbedding:
    """MLX affine int4 token embedding (`AffineQuantEmbedding`, crates/models/quantization/src/layers_quant.rs:105-150):
    a `[vocab, hidden]` table of 4-bit codes with a scale and an offset per group, gathered and dequantised in one
    pass (`scr_affine_b4_embed`).  The table is held as an `AffineQuantLinear` of N = vocab, K = hidden, so a tied
    lm_head is the same object and the same device buffer (the reference shares one buffer triple the same way)."""
    table: AffineQuantLinear

    # ---- MetalAffineEmbedOps::load (crates/targets/metal/src/layers_quant.rs:672-700)
    @classmethod
    def load(cls, weights: GpuWeights, prefix: str, group_size: int, bits: int) -> "AffineQuantEmbedding":
        if bits != 4:
            raise ScratchyCudaError(-4, f"bits={bits}: the quantized embedding exists at 4 bits only")
        # vocab and hidden come from the packed tensor's shape (hidden through the ceil(K * bits / 32) law), as in the reference
        hidden = int(weights.peek(f"{prefix}.weight").shape[1]) * 32 // bits
        return cls(AffineQuantLinear.load(weights, prefix, group_size, bits, hidden))

    @classmethod
    def from_tensors(cls, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, group_size: int = 64,
                     bits: int = 4) -> "AffineQuantEmbedding":
        return cls(AffineQuantLinear.from_tensors(weight, scales, biases, group_size, bits))

    @property
    def vocab_size(self) -> int:
        return self.table.out_features

    @property
    def hidden_size(self) -> int:
        return self.table.in_features

    def as_linear(self) -> AffineQuantLinear:
        """The tied lm_head: logits = x @ dequant(table)^T over the same buffer."""
        return self.table

    def forward(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        ids = ids.reshape(-1).contiguous()
        if ids.dtype not in (torch.int32, torch.uint32):
            raise ValueError(f"token ids must be 32-bit integers, got {ids.dtype}")
        n = int(ids.numel())
        dev = ids.device
        if out is None:
            out = torch.empty((n, self.hidden_size), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_affine_b4_embed(ctx.handle, _ptr(self.table.packed), _ptr(ids), n, self.vocab_size,
                                                 self.hidden_size, self.table.group_size, _ptr(out), _stream(dev)))
        return out


class AffineTape:
    """A static tape of int4 matvecs that runs as ONE launch (`scr_linear_affine_b4_tape`), the way the
    reference's decode step is a tape of dispatches fixed at build time
    (crates/targets/metal/src/tape/step.rs).  `jobs`: (linear, x [max_rows, K], y [max_rows, N], deps) in
    tape order; `deps` lists up to three earlier jobs that must have stored their output before this
    one starts — the producer of x and, when a buffer is reused, its earlier readers and writers.
    The tensors are bound for the life of the tape."""

    def __init__(self, jobs, max_rows: int = 1):
        if not jobs:
            raise ValueError("an empty tape")
        dev = jobs[0][1].device
        self._keep = []
        arr = (_lib.TapeLinear * len(jobs))()
        for j, (lin, x, y, deps) in enumerate(jobs):
            if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16 or not x.is_contiguous() or not y.is_contiguous():
                raise ValueError(f"tape job {j}: x and y must be contiguous bf16 tensors")
            if tuple(x.shape) != (max_rows, lin.in_features) or tuple(y.shape) != (max_rows, lin.out_features):
                raise ValueError(f"tape job {j}: x {tuple(x.shape)} / y {tuple(y.shape)} do not match "
                                 f"[{max_rows}, {lin.in_features}] / [{max_rows}, {lin.out_features}]")
            deps = list(deps)
            if len(deps) > 3:
                raise ValueError(f"tape job {j}: at most three dependencies")
            arr[j].packed, arr[j].x, arr[j].y = lin.packed.data_ptr(), x.data_ptr(), y.data_ptr()
            arr[j].N, arr[j].K, arr[j].group = lin.out_features, lin.in_features, lin.group_size
            for d in range(3):
                arr[j].dep[d] = int(deps[d]) if d < len(deps) else -1
            self._keep.append((lin, x, y))
        self.device, self.max_rows, self.n_jobs = dev, int(max_rows), len(jobs)
        self._ctx = _lib.context(_dev_index(dev))
        self._h = ctypes.c_void_p()
        torch.cuda.synchronize(dev)
        self._ctx.check(_lib.lib().scr_affine_b4_tape_create(self._ctx.handle, ctypes.cast(arr, ctypes.c_void_p), len(jobs),
                                                             int(max_rows), ctypes.byref(self._h)))

    def run(self, M: Optional[int] = None) -> None:
        """y_j = x_j @ W_j^T for every job, rows 0..M-1 (M defaults to max_rows), on the current stream."""
        self._ctx.check(_lib.lib().scr_linear_affine_b4_tape(self._ctx.handle, self._h, int(M or self.max_rows),
                                                             _stream(self.device)))

    def close(self) -> None:
        if self._h:
            _lib.lib().scr_tape_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _take_affine_scales(weights: GpuWeights, name: str) -> torch.Tensor:
    """`take_affine_scales` (layers_quant.rs:270-285): refuse scales that are not the pinned dtype."""
    compiled = weights.rmsnorm_scale_dtype()
    if compiled is None:
        raise ValueError(f"`{name}`: no scale dtype pinned")
    t = weights.take(name)
    if t.dtype != compiled:
        raise ValueError(f"`{name}` is {t.dtype} on disk; this build's quantized kernels read {compiled}")
    return t


@dataclass
class Fp8ActPack:
    """A per-token quantised activation (x_q, a_scale) that several linears may share."""
    buf: torch.Tensor
    M: int
    K: int

    def unpack(self):
        """Test hook: plain x_q [M,K] uint8 and a_scale [M] f32."""
        dev = self.buf.device
        xq = torch.empty((self.M, self.K), dtype=torch.uint8, device=dev)
        a = torch.empty((self.M,), dtype=torch.float32, device=dev)
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_fp8_act_unpack(ctx.handle, _ptr(self.buf), self.M, self.K, _ptr(xq), _ptr(a),
                                                _stream(dev)))
        return xq, a


@dataclass
class Fp8Linear:
    """fp8-dynamic-per-channel linear: e4m3 weights [N,K], f32 scale per output channel,
    activations quantised per token at run time (crates/layers/src/layers.rs:179-191)."""
    packed: torch.Tensor
    in_features: int
    out_features: int
    linear_bias: Optional[torch.Tensor] = None      # `{prefix}.bias` [N] bf16 (the q/k/v projections of Qwen2.5 carry one)

    @classmethod
    def load(cls, weights: GpuWeights, prefix: str, expected_in_features: int) -> "Fp8Linear":
        weight = weights.take(f"{prefix}.weight")
        scale = weights.take(f"{prefix}.weight_scale")
        linear_bias = weights.take(f"{prefix}.bias") if weights.contains(f"{prefix}.bias") else None
        if weight.dim() != 2 or int(weight.shape[1]) != expected_in_features:
            raise ValueError(f"`{prefix}.weight` is {tuple(weight.shape)}; this build expects "
                             f"in_features={expected_in_features}")
        return cls.from_tensors(weight, scale, linear_bias)

    @classmethod
    def from_tensors(cls, weight_e4m3: torch.Tensor, weight_scale: torch.Tensor,
                     linear_bias: Optional[torch.Tensor] = None) -> "Fp8Linear":
        if weight_e4m3.dtype not in (torch.uint8, torch.float8_e4m3fn):
            raise ValueError(f"`.weight` must be FP8 E4M3 bytes, got {weight_e4m3.dtype}")
        if not weight_e4m3.is_cuda:
            raise ScratchyCudaError(-5, "weights must be on a CUDA device (there is no CPU path)")
        N, K = int(weight_e4m3.shape[0]), int(weight_e4m3.shape[1])
        scale = weight_scale.reshape(-1).to(torch.float32).contiguous()   # [N] or [N,1] per-channel
        if scale.numel() != N:
            raise ValueError(f"`.weight_scale` must hold {N} per-channel scales, got {tuple(weight_scale.shape)}")
        dev = weight_e4m3.device
        ctx = _lib.context(_dev_index(dev))
        L = _lib.lib()
        size = ctypes.c_size_t(0)
        ctx.check(L.scr_fp8_repack_size(N, K, ctypes.byref(size)))
        packed = torch.empty(size.value, dtype=torch.uint8, device=dev)
        w = weight_e4m3.contiguous().view(torch.uint8)
        ctx.check(L.scr_fp8_repack(ctx.handle, _ptr(w), _ptr(scale), N, K, _ptr(packed), _stream(dev)))
        if linear_bias is not None:
            if linear_bias.dtype != torch.bfloat16 or tuple(linear_bias.shape) != (N,):
                raise ValueError(f"`.bias` must be bf16 [{N}], got {linear_bias.dtype} {tuple(linear_bias.shape)}")
            linear_bias = linear_bias.to(dev).contiguous()
        return cls(packed, K, N, linear_bias)

    @staticmethod
    def quantize_activation(x: torch.Tensor) -> Fp8ActPack:
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("x must be a bf16 CUDA tensor")
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M, K = int(x2.shape[0]), int(x2.shape[1])
        dev = x2.device
        ctx = _lib.context(_dev_index(dev))
        L = _lib.lib()
        size = ctypes.c_size_t(0)
        ctx.check(L.scr_fp8_act_size(M, K, ctypes.byref(size)))
        buf = torch.empty(size.value, dtype=torch.uint8, device=dev)
        ctx.check(L.scr_fp8_quant_per_token(ctx.handle, _ptr(x2), M, K, _ptr(buf), _stream(dev)))
        return Fp8ActPack(buf, M, K)

    @staticmethod
    def quantize_rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float,
                         normed_out: Optional[torch.Tensor] = None) -> Fp8ActPack:
        """RMSNorm and the per-token quantisation in one launch (`scr_rmsnorm_fp8_quant`): the pack that
        `quantize_activation(rmsnorm(x))` would give, plus (optionally) the bf16 normed rows."""
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        M, K = int(x2.shape[0]), int(x2.shape[1])
        dev = x2.device
        size = ctypes.c_size_t(0)
        st = _lib.lib().scr_fp8_act_size(M, K, ctypes.byref(size))
        if st:
            raise ScratchyCudaError(st, "scr_fp8_act_size")
        buf = torch.empty(size.value, dtype=torch.uint8, device=dev)
        ctx = _lib.context(_dev_index(dev))
        ctx.check(_lib.lib().scr_rmsnorm_fp8_quant(ctx.handle, _ptr(x2), _ptr(gain), ctypes.c_float(eps), M, K, _ptr(buf),
                                                   _ptr(normed_out), _stream(dev)))
        return Fp8ActPack(buf, M, K)

    def workspace_bytes(self, M: int) -> int:
        size = ctypes.c_size_t(0)
        st = _lib.lib().scr_linear_workspace_size(KIND_FP8_DYNAMIC, M, self.out_features, self.in_features,
                                                  ctypes.byref(size))
        if st:
            raise ScratchyCudaError(st, "scr_linear_workspace_size")
        return size.value

    def forward_quantized(self, act: Fp8ActPack, out: Optional[torch.Tensor] = None,
                          workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        if act.K != self.in_features:
            raise ValueError(f"activation has {act.K} features, layer expects {self.in_features}")
        dev = act.buf.device
        if out is None:
            out = torch.empty((act.M, self.out_features), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        need = self.workspace_bytes(act.M)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        ctx.check(_lib.lib().scr_linear_fp8(ctx.handle, _ptr(self.packed), _ptr(act.buf), act.M, self.out_features,
                                            self.in_features, _ptr(self.linear_bias), _ptr(out), _ptr(workspace),
                                            ctypes.c_size_t(workspace.numel()), _stream(dev)))
        return out

    def forward_partial(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                        workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-parallel use: quantise this rank's K-slice per token, unrounded f32 sums out
        (`scr_linear_fp8_dynamic_partial`)."""
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if out is None:
            out = torch.empty((M, self.out_features), dtype=torch.float32, device=dev)
        ctx = _lib.context(_dev_index(dev))
        need = self.workspace_bytes(M)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        ctx.check(_lib.lib().scr_linear_fp8_dynamic_partial(ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features,
                                                            self.in_features, _ptr(out), _ptr(workspace),
                                                            ctypes.c_size_t(workspace.numel()), _stream(dev)))
        return out

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The whole generated Linear: quantise per token, contract, dequantise (`scr_linear_fp8_dynamic`)."""
        if x.dtype != torch.bfloat16 or not x.is_cuda:
            raise ValueError("x must be a bf16 CUDA tensor")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"x has {x.shape[-1]} features, layer expects {self.in_features}")
        x2 = x.reshape(-1, self.in_features).contiguous()
        M = int(x2.shape[0])
        dev = x2.device
        if out is None:
            out = torch.empty((M, self.out_features), dtype=torch.bfloat16, device=dev)
        ctx = _lib.context(_dev_index(dev))
        need = self.workspace_bytes(M)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ctx.check(_lib.lib().scr_linear_fp8_dynamic(ctx.handle, _ptr(self.packed), _ptr(x2), M, self.out_features,
                                                    self.in_features, _ptr(self.linear_bias), _ptr(out), _ptr(workspace),
                                                    ctypes.c_size_t(workspace.numel()), _stream(dev)))
        return out.reshape(*x.shape[:-1], self.out_features)


class LinearLayer:
    """The variants of the reference's `LinearLayer` enum this target lowers
    (crates/layers/src/layers.rs:212-236): `AffineQuant` and `Fp8`."""

    AffineQuant = AffineQuantLinear
    Fp8 = Fp8Linear

    @staticmethod
    def load_affine_quant(weights: GpuWeights, prefix: str, group_size: int, bits: int,
                          expected_in_features: int) -> AffineQuantLinear:
        return AffineQuantLinear.load(weights, prefix, group_size, bits, expected_in_features)

    @staticmethod
    def load_fp8(weights: GpuWeights, prefix: str, expected_in_features: int) -> Fp8Linear:
        return Fp8Linear.load(weights, prefix, expected_in_features)


def load_layered_linear_affine_quant(gw: GpuWeights, n_layers: int, root: str, suffix: str, group_size: int,
                                     bits: int, in_features: int) -> List[AffineQuantLinear]:
    """crates/targets/metal/src/loaders.rs:96-116: one layer per `{root}.{i}.{suffix}`."""
    return [LinearLayer.load_affine_quant(gw, f"{root}.{i}.{suffix}", group_size, bits, in_features)
            for i in range(n_layers)]


def load_layered_linear_fp8_dynamic(gw: GpuWeights, n_layers: int, root: str, suffix: str,
                                    in_features: int) -> List[Fp8Linear]:
    """The `load_layered_fp8...` loader the reference's codegen names (no live target implements it)."""
    return [LinearLayer.load_fp8(gw, f"{root}.{i}.{suffix}", in_features) for i in range(n_layers)]
