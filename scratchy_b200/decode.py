"""One Llama decode step over the C ABI: the operators around the quantized linears and the step itself.

Host-side mirror of the reference's decode program (embed -> per layer [rmsnorm, fused QKV, RoPE +
paged-KV append, paged decode attention, o, residual add + rmsnorm, fused gate/up, silu*up, down] ->
final norm -> lm_head -> greedy argmax).  Up to 16 tokens silu*up runs as the epilogue of the gate/up matvec,
and RoPE + the cache append run inside the attention launch when the cache's blocks are multiples of 16 tokens.
The residual add + rmsnorm can run as the epilogue of the o / down matvecs too (`fuse_residual_norm=True`), but
that measured slower than the separate kernel (the ticket and the last CTA's serial pass cost more than the
launch they save), so it is off by default.  Each operator wrapper names the reference host golden it is
checked against (crates/targets/metal/src/cpu_golden.rs); the fused QKV and gate/up projections are
built with the reference's `load_rows_concat` law (crates/targets/metal/src/layers_quant.rs:363-450).

Every buffer of the step is allocated once in `DecodeBuffers`, so the step allocates nothing and
can be captured in a CUDA graph (`LlamaDecoder.capture`).  There is no CPU path.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import _lib, synth
from .layers import AffineQuantEmbedding, AffineQuantLinear, GpuWeights, _dev_index, _ptr, _stream


def _ctx(dev):
    return _lib.context(_dev_index(dev))


def _rows(t: torch.Tensor) -> int:
    """Row stride in elements of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("expected a 2-D tensor with dense rows")
    return int(t.stride(0))


# ------------------------------------------------------------------------------------ operators
def embed(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:114-124 (`embed`): out[i] = table[ids[i]]; ids are uint32 stored as int32."""
    dev = table.device
    n = int(ids.numel())
    if out is None:
        out = torch.empty((n, table.shape[1]), dtype=torch.bfloat16, device=dev)
    c = _ctx(dev)
    c.check(_lib.lib().scr_embed_bf16(c.handle, _ptr(ids), n, _ptr(table), int(table.shape[0]), int(table.shape[1]),
                                      _ptr(out), _stream(dev)))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:25-37 (`rmsnorm`) per row."""
    dev = x.device
    x2 = x.reshape(-1, x.shape[-1])
    if out is None:
        out = torch.empty_like(x2)
    c = _ctx(dev)
    c.check(_lib.lib().scr_rmsnorm_bf16(c.handle, _ptr(x2), _ptr(weight), _ptr(out), int(x2.shape[0]), int(x2.shape[1]),
                                        ctypes.c_float(eps), _stream(dev)))
    return out


def fused_add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:171-200 (`fused_add_rmsnorm`): residual += delta in place; returns rmsnorm(residual)."""
    dev = residual.device
    if out is None:
        out = torch.empty_like(residual)
    c = _ctx(dev)
    c.check(_lib.lib().scr_fused_add_rmsnorm_bf16(c.handle, _ptr(residual), _ptr(delta), _ptr(weight), _ptr(out),
                                                  int(residual.shape[0]), int(residual.shape[1]), ctypes.c_float(eps),
                                                  _stream(dev)))
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:211-219 (`fused_gate_up_silu_mul`); gate/up may be the halves of one fused output."""
    dev = gate.device
    ld = _rows(gate)
    if _rows(up) != ld:
        raise ValueError("gate and up must share a row stride")
    rows, inter = int(gate.shape[0]), int(gate.shape[1])
    if out is None:
        out = torch.empty((rows, inter), dtype=torch.bfloat16, device=dev)
    c = _ctx(dev)
    c.check(_lib.lib().scr_silu_mul_bf16(c.handle, _ptr(gate), _ptr(up), ld, _ptr(out), rows, inter, _stream(dev)))
    return out


def rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                cos_table: torch.Tensor, sin_table: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
                num_q_heads: int, num_kv_heads: int, head_dim: int, block_size: int,
                q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:289-362 (`rope_append`).  Caches are [num_blocks, num_kv_heads, block_size, head_dim]
    bf16; `q_out` defaults to q (in place)."""
    dev = q.device
    if q_out is None:
        q_out = q
    num_blocks = cache_k.numel() // (num_kv_heads * block_size * head_dim)
    c = _ctx(dev)
    c.check(_lib.lib().scr_rope_append_bf16(
        c.handle, _ptr(q), _rows(q), _ptr(k), _rows(k), _ptr(v), _rows(v), _ptr(positions), _ptr(slot_mapping),
        _ptr(cos_table), _ptr(sin_table), int(cos_table.shape[0]), _ptr(q_out), _rows(q_out), _ptr(cache_k), _ptr(cache_v),
        int(num_blocks), int(q.shape[0]), num_q_heads, num_kv_heads, head_dim, block_size, _stream(dev)))
    return q_out


def attention_via_cache(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, block_table: torch.Tensor,
                        seq_used_k: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, block_size: int,
                        attn_scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cpu_golden.rs:386-460 (`attention_via_cache`): one query token per sequence over the paged cache."""
    dev = q.device
    batch = int(q.shape[0])
    if out is None:
        out = torch.empty((batch, num_q_heads * head_dim), dtype=torch.bfloat16, device=dev)
    num_blocks = cache_k.numel() // (num_kv_heads * block_size * head_dim)
    c = _ctx(dev)
    c.check(_lib.lib().scr_attention_via_cache_bf16(
        c.handle, _ptr(q), _rows(q), _ptr(cache_k), _ptr(cache_v), int(num_blocks), _ptr(block_table), _ptr(seq_used_k),
        _ptr(out), _rows(out), batch, num_q_heads, num_kv_heads, head_dim, block_size, int(block_table.shape[1]),
        ctypes.c_float(attn_scale), _stream(dev)))
    return out


def rope_attention_via_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                             cos_table: torch.Tensor, sin_table: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor,
                             block_table: torch.Tensor, seq_used_k: torch.Tensor, num_q_heads: int, num_kv_heads: int,
                             head_dim: int, block_size: int, attn_scale: float,
                             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`rope_append` then `attention_via_cache` (cpu_golden.rs:289-362, 386-460) in one launch for a decode step.
    The new token of sequence b lands in the slot of token seq_used_k[b] - 1 (what the reference's slot_mapping
    names for it); q is left unrotated.  Raises SCR_E_UNSUPPORTED unless block_size is a multiple of 16 (<= 256)."""
    dev = q.device
    batch = int(q.shape[0])
    if out is None:
        out = torch.empty((batch, num_q_heads * head_dim), dtype=torch.bfloat16, device=dev)
    num_blocks = cache_k.numel() // (num_kv_heads * block_size * head_dim)
    c = _ctx(dev)
    c.check(_lib.lib().scr_rope_attention_via_cache_bf16(
        c.handle, _ptr(q), _rows(q), _ptr(k), _rows(k), _ptr(v), _rows(v), _ptr(positions), _ptr(cos_table), _ptr(sin_table),
        int(cos_table.shape[0]), _ptr(cache_k), _ptr(cache_v), int(num_blocks), _ptr(block_table), _ptr(seq_used_k),
        _ptr(out), _rows(out), batch, num_q_heads, num_kv_heads, head_dim, block_size, int(block_table.shape[1]),
        ctypes.c_float(attn_scale), _stream(dev)))
    return out


def rope_attention_supported(block_size: int) -> bool:
    """Geometries for which the one-launch RoPE + append + attention exists."""
    return block_size % 16 == 0 and block_size <= 256


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row: largest value, smallest id among equal ones, NaN never
    (crates/targets/metal/tests/argmax_split_test.rs:24-33).  Returns uint32 ids stored as int32."""
    dev = logits.device
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=dev)
    c = _ctx(dev)
    c.check(_lib.lib().scr_argmax_bf16(c.handle, _ptr(logits), _rows(logits), int(logits.shape[0]), int(logits.shape[1]),
                                       _ptr(out), _stream(dev)))
    return out


# ------------------------------------------------------------------------------------ model
@dataclass(frozen=True)
class LlamaConfig:
    hidden: int
    n_layers: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    group_size: int = 64

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


LLAMA_3_2_3B = LlamaConfig(hidden=3072, n_layers=28, n_q_heads=24, n_kv_heads=8, head_dim=128, intermediate=8192,
                           vocab=128256)


def rope_tables(max_pos: int, head_dim: int, theta: float):
    """f32 cos/sin tables [max_pos, head_dim]; the kernels read the first head_dim/2 columns of a row
    (the second half repeats the first, as the checkpoint-side convention stores them)."""
    half = head_dim // 2
    inv_freq = (1.0 / (theta ** (np.arange(half, dtype=np.float64) * 2.0 / head_dim)))
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv_freq[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1).astype(np.float32)
    return cos, sin


def synthetic_checkpoint(cfg: LlamaConfig, seed: int = 0) -> dict:
    """Random-init weights with the benchmark's int4 distributions (numpy, host): per layer the seven
    projections as (codes, scales, biases), bf16 norm gains, a bf16 embedding table and an int4 lm_head."""
    rng = np.random.default_rng(synth.seed_for("llama-decode", cfg.hidden, cfg.n_layers, seed))
    ck = {}

    def put_linear(prefix, n, k, s):
        w, sc, b = synth.affine_int4_weights(n, k, cfg.group_size, seed=s)
        ck[f"{prefix}.weight"], ck[f"{prefix}.scales"], ck[f"{prefix}.biases"] = w, sc, b

    def gain(n):
        return synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32))

    for i in range(cfg.n_layers):
        root = f"model.layers.{i}"
        s = synth.seed_for("llama-decode-layer", i, seed)
        put_linear(f"{root}.self_attn.q_proj", cfg.q_dim, cfg.hidden, s + 1)
        put_linear(f"{root}.self_attn.k_proj", cfg.kv_dim, cfg.hidden, s + 2)
        put_linear(f"{root}.self_attn.v_proj", cfg.kv_dim, cfg.hidden, s + 3)
        put_linear(f"{root}.self_attn.o_proj", cfg.hidden, cfg.q_dim, s + 4)
        put_linear(f"{root}.mlp.gate_proj", cfg.intermediate, cfg.hidden, s + 5)
        put_linear(f"{root}.mlp.up_proj", cfg.intermediate, cfg.hidden, s + 6)
        put_linear(f"{root}.mlp.down_proj", cfg.hidden, cfg.intermediate, s + 7)
        ck[f"{root}.input_layernorm.weight"] = gain(cfg.hidden)
        ck[f"{root}.post_attention_layernorm.weight"] = gain(cfg.hidden)
    ck["model.norm.weight"] = gain(cfg.hidden)
    ck["model.embed_tokens.weight"] = synth.f32_to_bf16_bits(
        (0.02 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(np.float32))
    put_linear("lm_head", cfg.vocab, cfg.hidden, synth.seed_for("llama-decode-head", seed))
    return ck


def synthetic_checkpoint_on_device(cfg: LlamaConfig, device, seed: int = 0) -> dict:
    """The same random-init checkpoint drawn with the device generator (full-size models: seconds, not minutes)."""
    g = torch.Generator(device=device)
    g.manual_seed(synth.seed_for("llama-decode-device", cfg.hidden, cfg.n_layers, seed))
    ck = {}

    def put_linear(prefix, n, k):
        ck[f"{prefix}.weight"] = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device=device,
                                               generator=g)
        sc = (torch.randn((n, k // cfg.group_size), device=device, generator=g) * 0.02).abs().add(1e-3).to(torch.bfloat16)
        ck[f"{prefix}.scales"] = sc
        ck[f"{prefix}.biases"] = (-8.0 * sc.float() + torch.randn((n, k // cfg.group_size), device=device, generator=g)
                                  * 1e-3).to(torch.bfloat16)

    def gain(n):
        return (1.0 + 0.1 * torch.randn(n, device=device, generator=g)).to(torch.bfloat16)

    for i in range(cfg.n_layers):
        root = f"model.layers.{i}"
        put_linear(f"{root}.self_attn.q_proj", cfg.q_dim, cfg.hidden)
        put_linear(f"{root}.self_attn.k_proj", cfg.kv_dim, cfg.hidden)
        put_linear(f"{root}.self_attn.v_proj", cfg.kv_dim, cfg.hidden)
        put_linear(f"{root}.self_attn.o_proj", cfg.hidden, cfg.q_dim)
        put_linear(f"{root}.mlp.gate_proj", cfg.intermediate, cfg.hidden)
        put_linear(f"{root}.mlp.up_proj", cfg.intermediate, cfg.hidden)
        put_linear(f"{root}.mlp.down_proj", cfg.hidden, cfg.intermediate)
        ck[f"{root}.input_layernorm.weight"] = gain(cfg.hidden)
        ck[f"{root}.post_attention_layernorm.weight"] = gain(cfg.hidden)
    ck["model.norm.weight"] = gain(cfg.hidden)
    ck["model.embed_tokens.weight"] = (0.02 * torch.randn((cfg.vocab, cfg.hidden), device=device, generator=g)).to(
        torch.bfloat16)
    put_linear("lm_head", cfg.vocab, cfg.hidden)
    return ck


def _to_device(arr, dev) -> torch.Tensor:
    if isinstance(arr, torch.Tensor):
        return arr.to(dev)
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16)).to(dev).view(torch.bfloat16)
    if arr.dtype == np.uint32:
        return torch.from_numpy(arr.view(np.int32)).to(dev)
    return torch.from_numpy(arr).to(dev)


@dataclass
class DecoderLayer:
    qkv: AffineQuantLinear
    o: AffineQuantLinear
    gate_up: AffineQuantLinear
    down: AffineQuantLinear
    input_norm: torch.Tensor
    post_norm: torch.Tensor


class PagedKvCache:
    """Per layer one K and one V buffer [num_blocks, num_kv_heads, block_size, head_dim] bf16
    (crates/targets/metal/src/paged_kv_layout.rs:1-60; the layer index is not part of the layout)."""

    def __init__(self, cfg: LlamaConfig, num_blocks: int, block_size: int, device):
        self.num_blocks, self.block_size = num_blocks, block_size
        shape = (num_blocks, cfg.n_kv_heads, block_size, cfg.head_dim)
        self.k = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.n_layers)]
        self.v = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.n_layers)]

    def nbytes(self) -> int:
        return sum(t.numel() * 2 for t in self.k) * 2


class DecodeBuffers:
    """Everything one step writes, for a fixed batch: allocated once so the step allocates nothing."""

    def __init__(self, cfg: LlamaConfig, batch: int, max_blocks_per_seq: int, device, workspace_bytes: int):
        bf, i32 = torch.bfloat16, torch.int32
        self.batch = batch
        self.ids = torch.zeros(batch, dtype=i32, device=device)
        self.positions = torch.zeros(batch, dtype=i32, device=device)
        self.slot_mapping = torch.zeros(batch, dtype=i32, device=device)
        self.block_table = torch.zeros((batch, max_blocks_per_seq), dtype=i32, device=device)
        self.seq_used_k = torch.zeros(batch, dtype=i32, device=device)
        self.residual = torch.empty((batch, cfg.hidden), dtype=bf, device=device)
        self.normed = torch.empty((batch, cfg.hidden), dtype=bf, device=device)
        self.qkv = torch.empty((batch, cfg.q_dim + 2 * cfg.kv_dim), dtype=bf, device=device)
        self.attn = torch.empty((batch, cfg.q_dim), dtype=bf, device=device)
        self.delta = torch.empty((batch, cfg.hidden), dtype=bf, device=device)
        self.gate_up = torch.empty((batch, 2 * cfg.intermediate), dtype=bf, device=device)
        self.act = torch.empty((batch, cfg.intermediate), dtype=bf, device=device)
        self.logits = torch.empty((batch, cfg.vocab), dtype=bf, device=device)
        self.next_ids = torch.zeros(batch, dtype=i32, device=device)
        self.workspace = torch.empty(max(workspace_bytes, 16), dtype=torch.uint8, device=device)
        # ticket counter + per-CTA sums of the fused residual/norm epilogue: zero once, the kernel keeps it zero
        self.ends_scratch = torch.zeros(AffineQuantLinear.ENDS_SCRATCH_BYTES, dtype=torch.uint8, device=device)


class LlamaDecoder:
    """Random-init or checkpoint-loaded Llama decoder whose every linear is MLX affine int4 g64."""

    def __init__(self, cfg: LlamaConfig, checkpoint, device, max_pos: int = 4096, fuse_residual_norm: bool = False,
                 fuse_rope: bool = True, fuse_ends: bool = False, exact_norm_in: bool = False, fuse_residual: bool = True):
        """`checkpoint`: a `GpuWeights` (e.g. `CheckpointWeights.from_dir(...)`) or a dict of host / device
        tensors with the HF Llama names.  `fuse_rope`: run RoPE + cache append inside the attention launch where
        the cache geometry allows it (the new token's slot is then taken from block_table / seq_used_k, which a
        decode step keeps consistent with slot_mapping).  `fuse_ends`: for the few tokens whose normalised rows fit the
        matvec's shared memory, run every RMSNorm inside the matvec that consumes it and every residual add inside the
        matvec that produces its summand (the reference's `QmvEnds`): five launches per layer instead of seven.  The
        residual adds keep the bits of the separate operator; the norm-in end runs the reference matvec's own arithmetic
        (the dot over `x * gain`, the row scaled by `1 / rms(x)`: as close to the exact product as norm-then-matvec, not
        its bits) unless `exact_norm_in` asks for the rounded normalised row of the separate RMSNorm (slower: every
        CTA then finishes the row's sum of squares before its first product).  `fuse_residual` (up to 16 tokens, when
        `fuse_ends` is off): the o and down projections add into the residual stream themselves (the residual end alone,
        the bits of the separate add) and the norms run as plain RMSNorm launches — the same number of launches as with
        `fused_add_rmsnorm`, each norm reading one row instead of two and no intermediate projection output."""
        if not torch.cuda.is_available():
            raise _lib.ScratchyCudaError(-5, "LlamaDecoder needs a CUDA device (there is no CPU path)")
        self.cfg, self.device = cfg, torch.device(device)
        self.fuse_residual_norm = fuse_residual_norm
        self.fuse_rope = fuse_rope
        self.fuse_ends = fuse_ends
        self.exact_norm_in = exact_norm_in
        self.fuse_residual = fuse_residual
        dev = self.device
        gw = checkpoint if isinstance(checkpoint, GpuWeights) else GpuWeights({k: _to_device(v, dev)
                                                                              for k, v in checkpoint.items()})
        g, h = cfg.group_size, cfg.hidden
        self.layers: List[DecoderLayer] = []
        for i in range(cfg.n_layers):
            root = f"model.layers.{i}"
            qkv = AffineQuantLinear.load_rows_concat(
                gw, [f"{root}.self_attn.q_proj", f"{root}.self_attn.k_proj", f"{root}.self_attn.v_proj"], g, 4, h)
            o = AffineQuantLinear.load(gw, f"{root}.self_attn.o_proj", g, 4, cfg.q_dim)
            gate_up = AffineQuantLinear.load_rows_interleave8(gw, f"{root}.mlp.gate_proj", f"{root}.mlp.up_proj", g, 4, h)
            down = AffineQuantLinear.load(gw, f"{root}.mlp.down_proj", g, 4, cfg.intermediate)
            for part in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "mlp.gate_proj", "mlp.up_proj"):
                for suffix in ("weight", "scales", "biases"):
                    gw.take(f"{root}.{part}.{suffix}")          # the fused projections are built: drop the parts
            self.layers.append(DecoderLayer(qkv, o, gate_up, down, gw.take(f"{root}.input_layernorm.weight"),
                                            gw.take(f"{root}.post_attention_layernorm.weight")))
        self.final_norm = gw.take("model.norm.weight")
        # `model.embed_tokens` with (weight = U32, scales, biases) is an `AffineQuantEmbedding`; without an `lm_head` of
        # its own the vocabulary head is tied to it and multiplies with the same buffer (the macro's rule,
        # crates/models/quantization/src/layers_quant.rs:105-126)
        self.quant_embed = None
        if gw.contains("model.embed_tokens.scales"):
            self.quant_embed = AffineQuantEmbedding.load(gw, "model.embed_tokens", g, 4)
            self.embed_table = None
        else:
            self.embed_table = gw.take("model.embed_tokens.weight")
        if gw.contains("lm_head.weight"):
            self.lm_head = AffineQuantLinear.load(gw, "lm_head", g, 4, h)
        elif self.quant_embed is not None:
            self.lm_head = self.quant_embed.as_linear()
        else:
            raise KeyError("tensor `lm_head.weight` not found in checkpoint (and no quantized embedding to tie it to)")
        for t in [self.final_norm] + ([self.embed_table] if self.embed_table is not None else []) + \
                [x for l in self.layers for x in (l.input_norm, l.post_norm)]:
            if t.dtype != torch.bfloat16:
                raise ValueError("norm gains and the embedding table must be bf16 for this build")
        cos, sin = rope_tables(max_pos, cfg.head_dim, cfg.rope_theta)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        self.attn_scale = 1.0 / math.sqrt(cfg.head_dim)
        torch.cuda.synchronize(dev)

    # ---- sizes
    def weight_bytes(self) -> int:
        """Bytes of packed linear weights one step streams (all layers + lm_head)."""
        n = sum(l.qkv.packed.numel() + l.o.packed.numel() + l.gate_up.packed.numel() + l.down.packed.numel()
                for l in self.layers)
        return n + self.lm_head.packed.numel()

    def workspace_bytes(self, batch: int) -> int:
        lins = [self.lm_head] + [x for l in self.layers for x in (l.qkv, l.o, l.gate_up, l.down)]
        return max(x.workspace_bytes(batch) for x in lins)

    def buffers(self, batch: int, max_blocks_per_seq: int) -> DecodeBuffers:
        return DecodeBuffers(self.cfg, batch, max_blocks_per_seq, self.device, self.workspace_bytes(batch))

    # ---- one step: reads buf.ids/positions/slot_mapping/block_table/seq_used_k, writes buf.logits/next_ids
    @staticmethod
    def _linear(lin, x: torch.Tensor, out: torch.Tensor, buf: DecodeBuffers) -> torch.Tensor:
        """A linear of the step: up to 16 tokens through the matvec-ends entry point (no end set here; the same kernel as
        `forward`), above through `forward` with the step's workspace."""
        if buf.batch <= 16 and isinstance(lin, AffineQuantLinear):
            return lin.forward_ends(x, out)
        return lin.forward(x, out=out, workspace=buf.workspace)

    def step(self, buf: DecodeBuffers, cache: PagedKvCache) -> torch.Tensor:
        cfg = self.cfg
        qd, kd = cfg.q_dim, cfg.kv_dim
        if self.quant_embed is not None:
            self.quant_embed.forward(buf.ids, out=buf.residual)
        else:
            embed(buf.ids, self.embed_table, out=buf.residual)
        ends = (self.fuse_ends and not self.fuse_residual_norm and
                AffineQuantLinear.norm_in_supported(buf.batch, cfg.hidden))
        row_scale = not self.exact_norm_in
        resid_end = self.fuse_residual and not ends and not self.fuse_residual_norm and buf.batch <= 16
        if not ends:
            rmsnorm(buf.residual, self.layers[0].input_norm, cfg.rms_eps, out=buf.normed)
        for i, layer in enumerate(self.layers):
            if ends:
                layer.qkv.forward_ends(buf.residual, buf.qkv, norm_gain=layer.input_norm, norm_eps=cfg.rms_eps,
                                       norm_row_scale=row_scale)
            else:
                self._linear(layer.qkv, buf.normed, buf.qkv, buf)
            q, k, v = buf.qkv[:, :qd], buf.qkv[:, qd:qd + kd], buf.qkv[:, qd + kd:]
            if self.fuse_rope and rope_attention_supported(cache.block_size):
                rope_attention_via_cache(q, k, v, buf.positions, self.cos, self.sin, cache.k[i], cache.v[i], buf.block_table,
                                         buf.seq_used_k, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cache.block_size,
                                         self.attn_scale, out=buf.attn)
            else:
                rope_append(q, k, v, buf.positions, buf.slot_mapping, self.cos, self.sin, cache.k[i], cache.v[i],
                            cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cache.block_size)
                attention_via_cache(q, cache.k[i], cache.v[i], buf.block_table, buf.seq_used_k, cfg.n_q_heads,
                                    cfg.n_kv_heads, cfg.head_dim, cache.block_size, self.attn_scale, out=buf.attn)
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
            if ends:
                # residual += o(attn); act = silu(gate) * up of rmsnorm(residual); residual += down(act)
                layer.o.forward_ends(buf.attn, buf.residual, residual=True)
                layer.gate_up.forward_ends(buf.residual, buf.act, norm_gain=layer.post_norm, norm_eps=cfg.rms_eps, silu_pairs=True,
                                           norm_row_scale=row_scale)
                layer.down.forward_ends(buf.act, buf.residual, residual=True)
            elif resid_end:
                layer.o.forward_ends(buf.attn, buf.residual, residual=True)
                rmsnorm(buf.residual, layer.post_norm, cfg.rms_eps, out=buf.normed)
                layer.gate_up.forward_silu_mul(buf.normed, out=buf.act, scratch=buf.gate_up, workspace=buf.workspace)
                layer.down.forward_ends(buf.act, buf.residual, residual=True)
                rmsnorm(buf.residual, nxt, cfg.rms_eps, out=buf.normed)
            elif self.fuse_residual_norm:
                layer.o.forward_residual_rmsnorm(buf.attn, buf.residual, layer.post_norm, cfg.rms_eps, buf.normed,
                                                 buf.ends_scratch, delta=buf.delta, workspace=buf.workspace)
                layer.gate_up.forward_silu_mul(buf.normed, out=buf.act, scratch=buf.gate_up, workspace=buf.workspace)
                layer.down.forward_residual_rmsnorm(buf.act, buf.residual, nxt, cfg.rms_eps, buf.normed, buf.ends_scratch,
                                                    delta=buf.delta, workspace=buf.workspace)
            else:
                self._linear(layer.o, buf.attn, buf.delta, buf)
                fused_add_rmsnorm(buf.residual, buf.delta, layer.post_norm, cfg.rms_eps, out=buf.normed)
                layer.gate_up.forward_silu_mul(buf.normed, out=buf.act, scratch=buf.gate_up, workspace=buf.workspace)
                self._linear(layer.down, buf.act, buf.delta, buf)
                fused_add_rmsnorm(buf.residual, buf.delta, nxt, cfg.rms_eps, out=buf.normed)
        if ends:
            self.lm_head.forward_ends(buf.residual, buf.logits, norm_gain=self.final_norm, norm_eps=cfg.rms_eps,
                                      norm_row_scale=row_scale)
        else:
            self._linear(self.lm_head, buf.normed, buf.logits, buf)
        argmax(buf.logits, out=buf.next_ids)
        return buf.logits

    def check_health(self) -> None:
        """Synchronise and raise `ScratchyCudaError` if a device-side check fired since the last call: a token id,
        position, slot or block id out of range (`SCR_E_ARG`; the access was skipped, the step's results are not to be
        used) or a bounded wait that ran out (`SCR_E_TIMEOUT`).  The word is read and cleared (`scr_device_status`); a
        serving loop calls this once per step, after it has synchronised on the step's tokens anyway — while the word is
        set every bounded wait on the context gives up early."""
        _ctx(self.device).device_status(None)

    def capture(self, buf: DecodeBuffers, cache: PagedKvCache) -> torch.cuda.CUDAGraph:
        """The whole step as one CUDA graph (warm once outside the capture first)."""
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self.step(buf, cache)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            self.step(buf, cache)
        return graph
