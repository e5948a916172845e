"""Tensor-parallel sharding of the quantized linears — host-side mirror of the reference's law.

Reference (paths relative to its root):
  * world typing            crates/core/tp-world/src/lib.rs:19-125 (`TpWorld<N>`, `Rank`)
  * slice law               crates/compiler/subtile/src/tensor_parallel.rs:1172-1240 (`slice_source`):
                            a whole activation splits the weight's output channels (`SourceShard::Cols`
                            of the `[K,N]` view = row blocks of the on-disk `[N,K]`; a per-channel scale
                            follows N); a column-split activation splits the contraction
                            (`SourceShard::Rows` of `[K,N]` = column blocks of `[N,K]`; scale whole; the
                            affine preset needs `(K/W) % group == 0`, :534-537) and leaves a `Partial`
  * collective meaning      tensor_parallel.rs:1342-1393 (`eval_collective`): AllReduce sums the ranks'
                            operands; the reference's host evaluator does it in rank order in f32

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in the CPU tests) is the plumbing.
The per-rank linears are the ordinary `AffineQuantLinear` / `Fp8Linear` over the sliced tensors:
slicing happens on the checkpoint tensors, before the load-time repack.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

VALID_WORLDS = (1, 2, 4, 8)          # the build features tp-2/4/8 of crates/core/tp-world/Cargo.toml:18-24


@dataclass(frozen=True)
class TpWorld:
    """`TpWorld<N>` + `Rank`: a world size from {1,2,4,8} and this process's rank in it."""
    world: int
    rank: int

    def __post_init__(self):
        if self.world not in VALID_WORLDS:
            raise ValueError(f"tensor-parallel world must be one of {VALID_WORLDS}, got {self.world}")
        if not 0 <= self.rank < self.world:
            raise ValueError(f"rank {self.rank} outside world {self.world}")


def slice_rows(full: torch.Tensor, tp: TpWorld) -> torch.Tensor:
    """Rank's block of rows of a 2-D (or 1-D, per-row) tensor: `full[r*lr:(r+1)*lr]`."""
    n = full.shape[0]
    if n % tp.world != 0:
        raise ValueError(f"{n} rows do not split over {tp.world} ranks")
    lr = n // tp.world
    return full[tp.rank * lr:(tp.rank + 1) * lr].contiguous()


def slice_cols(full: torch.Tensor, tp: TpWorld, unit: int = 1) -> torch.Tensor:
    """Rank's block of columns of a 2-D tensor; `unit` = logical elements per stored column
    (8 for U32-packed int4 codes, 64 for per-group scales)."""
    c = full.shape[1]
    if c % tp.world != 0:
        raise ValueError(f"{c * unit} columns do not split over {tp.world} ranks")
    lc = c // tp.world
    return full[:, tp.rank * lc:(tp.rank + 1) * lc].contiguous()


# ---------------------------------------------------------------------------- affine int4
def shard_affine_column_parallel(weight, scales, biases, tp: TpWorld):
    """q/k/v/gate/up: split the output channels (rows of `[N, K/8]`, `[N, K/64]`)."""
    return slice_rows(weight, tp), slice_rows(scales, tp), slice_rows(biases, tp)


def shard_affine_row_parallel(weight, scales, biases, tp: TpWorld, group_size: int = 64):
    """o/down: split the contraction (columns).  Refused unless `(K/W) % group == 0`
    (tensor_parallel.rs:534-537)."""
    K = weight.shape[1] * 8
    if (K // tp.world) % group_size != 0 or K % tp.world != 0:
        raise ValueError(f"K={K} over {tp.world} ranks leaves {K / tp.world} per rank, not a multiple of "
                         f"group_size={group_size}")
    return slice_cols(weight, tp, 8), slice_cols(scales, tp, group_size), slice_cols(biases, tp, group_size)


# ---------------------------------------------------------------------------- fp8 per-channel
def shard_fp8_column_parallel(weight_e4m3, weight_scale, tp: TpWorld):
    return slice_rows(weight_e4m3, tp), slice_rows(weight_scale.reshape(-1), tp)


def shard_fp8_row_parallel(weight_e4m3, weight_scale, tp: TpWorld):
    """The per-channel scale stays whole; each rank quantises its own K-slice of the activation
    per token, so `a_scale` differs per rank and the partials are dequantised before the sum."""
    return slice_cols(weight_e4m3, tp), weight_scale.reshape(-1).contiguous()


# ---------------------------------------------------------------------------- collective
class TpCommunicator:
    """The `SubOp::AllReduce` of a row-parallel layer: a sum over the ranks of a process group."""

    def __init__(self, tp: TpWorld, group: Optional[dist.ProcessGroup] = None):
        self.tp = tp
        self.group = group
        if tp.world > 1:
            if not dist.is_initialized():
                raise RuntimeError("torch.distributed is not initialised")
            ws = dist.get_world_size(group)
            if ws != tp.world:
                raise ValueError(f"process group has {ws} ranks, TpWorld says {tp.world}")

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_gather_cols(self, local: torch.Tensor, cols: int) -> torch.Tensor:
        """The `SubOp::AllGather{cols}` of an N-split layer (crates/compiler/subtile/src/tensor_parallel.rs:1363-1386):
        the ranks' [rows, lc] column blocks side by side in rank order, cropped to `cols`."""
        rows, lc = local.shape
        if lc * self.tp.world < cols:
            raise ValueError(f"{self.tp.world} blocks of {lc} columns cannot restore {cols}")
        if self.tp.world == 1:
            return local[:, :cols].contiguous()
        blocks = [torch.empty_like(local) for _ in range(self.tp.world)]
        dist.all_gather(blocks, local.contiguous(), group=self.group)
        return torch.cat(blocks, dim=1)[:, :cols].contiguous()


class OneShotAllReduce:
    """The decode-size exchange: `scr_tp_allreduce_partial`, one kernel per rank over NVLink peer memory,
    rank-ordered f32 sum and a single rounding (the reference's meaning of AllReduce, bit for bit).
    Creating it allocates the rank's receive buffer and exchanges the IPC handles through the process
    group; every rank must then issue the same sequence of calls."""

    def __init__(self, tp: TpWorld, device, max_elems: int, group: Optional[dist.ProcessGroup] = None,
                 connect: bool = True):
        """`connect=False` leaves the peers unconnected: ranks that are threads of one process then call
        `connect_local` on each other (an IPC handle opens only in another process)."""
        import ctypes
        from . import _lib
        self.tp, self.max_elems = tp, int(max_elems)
        self.device = torch.device(device)
        self._lib = _lib
        self._ctx = _lib.context(self.device.index if self.device.index is not None else torch.cuda.current_device())
        self._h = ctypes.c_void_p()
        handle = (ctypes.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            self._ctx.check(_lib.lib().scr_tp_comm_create(self._ctx.handle, tp.world, tp.rank, self.max_elems,
                                                          ctypes.byref(self._h), handle))
            if tp.world > 1 and connect:
                if not dist.is_initialized():
                    raise RuntimeError("torch.distributed is not initialised")
                gathered = [None] * tp.world
                dist.all_gather_object(gathered, bytes(handle), group=group)
                blob = (ctypes.c_uint8 * (64 * tp.world)).from_buffer_copy(b"".join(gathered))
                self._ctx.check(_lib.lib().scr_tp_comm_connect(self._h, blob))
                dist.barrier(group=group)
        self._group = group

    @property
    def base(self) -> int:
        """Device address of this rank's receive buffer (`scr_tp_comm_base`), what in-process peers connect to."""
        import ctypes
        b = ctypes.c_void_p()
        self._ctx.check(self._lib.lib().scr_tp_comm_base(self._h, ctypes.byref(b)))
        return int(b.value)

    def connect_local(self, bases, devices) -> None:
        """`scr_tp_comm_connect_local`: ranks as threads of one process (the reference's `ThreadPoolExecutor`,
        crates/serving/worker/src/threadpool.rs:1-16) connect through raw device pointers; `bases[r]`,
        `devices[r]` = rank r's `base` and device index.  Call with this rank's device current."""
        import ctypes
        arr = (ctypes.c_void_p * self.tp.world)(*[ctypes.c_void_p(int(b)) for b in bases])
        dev = (ctypes.c_int32 * self.tp.world)(*[int(d) for d in devices])
        with torch.cuda.device(self.device):
            self._ctx.check(self._lib.lib().scr_tp_comm_connect_local(self._h, arr, dev))

    def set_wait_limit(self, polls: int) -> None:
        """`scr_tp_comm_set_wait_limit`: polls before a kernel of this communicator gives up on a peer."""
        self._ctx.check(self._lib.lib().scr_tp_comm_set_wait_limit(self._h, int(polls)))

    def check_health(self) -> None:
        """Synchronise and raise `ScratchyCudaError(SCR_E_TIMEOUT)` if a bounded wait ran out since the last
        check (`scr_device_status`; the reference's `Executor::check_health`).  Call it once per step, after the
        host has synchronised on the step's result anyway: while the status word is set every bounded wait on
        this context gives up early."""
        self._ctx.device_status(None)

    def all_reduce(self, part: torch.Tensor, out_bf16: Optional[torch.Tensor] = None,
                   out_f32: Optional[torch.Tensor] = None) -> torch.Tensor:
        """f32 partials in; the reduced values as bf16 (default) and/or f32 out."""
        import ctypes
        if part.dtype != torch.float32 or not part.is_cuda or not part.is_contiguous():
            raise ValueError("partials must be a contiguous f32 CUDA tensor")
        if out_bf16 is None and out_f32 is None:
            out_bf16 = torch.empty(part.shape, dtype=torch.bfloat16, device=part.device)
        self._ctx.check(self._lib.lib().scr_tp_allreduce_partial(
            self._h, ctypes.c_void_p(part.data_ptr()), part.numel(),
            ctypes.c_void_p(out_bf16.data_ptr()) if out_bf16 is not None else None,
            ctypes.c_void_p(out_f32.data_ptr()) if out_f32 is not None else None,
            ctypes.c_void_p(torch.cuda.current_stream(part.device).cuda_stream)))
        return out_bf16 if out_bf16 is not None else out_f32

    def all_gather_cols(self, local: torch.Tensor, cols: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`scr_tp_allgather_cols`: the ranks' [rows, lc] bf16 column blocks side by side in rank order, cropped to
        `cols`, on every rank, as one launch over peer memory."""
        import ctypes
        if local.dtype != torch.bfloat16 or not local.is_cuda or not local.is_contiguous() or local.dim() != 2:
            raise ValueError("the column block must be a contiguous 2-D bf16 CUDA tensor")
        rows, lc = (int(v) for v in local.shape)
        if out is None:
            out = torch.empty((rows, cols), dtype=torch.bfloat16, device=local.device)
        self._ctx.check(self._lib.lib().scr_tp_allgather_cols(
            self._h, ctypes.c_void_p(local.data_ptr()), rows, lc, int(cols), ctypes.c_void_p(out.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream(local.device).cuda_stream)))
        return out

    def fp8_linear_all_reduce(self, linear, x_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """A row-parallel `Fp8Linear` and its all-reduce as one launch (`scr_linear_fp8_dynamic_allreduce`):
        the same bits as `linear.forward_partial` followed by `all_reduce`.  Raises SCR_E_UNSUPPORTED beyond
        the self-quantising matvec (a few tokens); see `fp8_linear_all_reduce_supported`."""
        import ctypes
        x2 = x_local.reshape(-1, linear.in_features).contiguous()
        M = int(x2.shape[0])
        if out is None:
            out = torch.empty((M, linear.out_features), dtype=torch.bfloat16, device=x2.device)
        self._ctx.check(self._lib.lib().scr_linear_fp8_dynamic_allreduce(
            self._h, ctypes.c_void_p(linear.packed.data_ptr()), ctypes.c_void_p(x2.data_ptr()), M, linear.out_features,
            linear.in_features, ctypes.c_void_p(out.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream(x2.device).cuda_stream)))
        return out

    def fp8_linear_all_reduce_supported(self, linear, M: int) -> bool:
        k16 = (linear.in_features + 15) // 16 * 16
        one_shot = min(self.max_elems, 524288)        # TPC_ONE_SHOT_MAX: capacity of the packet area
        return M <= 4 and linear.in_features % 8 == 0 and M * k16 <= 14 * 1024 and M * linear.out_features <= one_shot

    def close(self) -> None:
        if self._h:
            if self.tp.world > 1 and dist.is_initialized():
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self._group)           # nobody frees a buffer a peer may still write
            self._lib.lib().scr_tp_comm_destroy(self._h)
            self._h = None


def partial_to_bf16(part: torch.Tensor) -> torch.Tensor:
    """`scr_partial_to_bf16`: the single rounding after the all-reduce."""
    import ctypes
    from . import _lib
    dev = part.device
    out = torch.empty(part.shape, dtype=torch.bfloat16, device=dev)
    ctx = _lib.context(dev.index if dev.index is not None else torch.cuda.current_device())
    ctx.check(_lib.lib().scr_partial_to_bf16(ctx.handle, ctypes.c_void_p(part.data_ptr()), part.numel(),
                                             ctypes.c_void_p(out.data_ptr()),
                                             ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return out


class RowParallel:
    """A row-parallel linear (o, down): local contraction over the rank's K-slice, then the all-reduce.
    With a `OneShotAllReduce` the exchange of decode-size outputs is one kernel over peer memory;
    larger outputs (prefill) go through the process group's all-reduce."""

    def __init__(self, linear, comm: TpCommunicator, one_shot: Optional[OneShotAllReduce] = None):
        self.linear = linear
        self.comm = comm
        self.one_shot = one_shot

    def forward(self, x_local: torch.Tensor, workspace=None) -> torch.Tensor:
        """f32 partials over the rank's K-slice, summed over ranks, rounded to bf16 once."""
        part = self.linear.forward_partial(x_local, workspace=workspace)
        n = part.numel()
        if self.one_shot is not None and n <= self.one_shot.max_elems and (
                (n <= 524288 and n % 4 == 0) or (n >= 131072 and n % (8 * self.comm.tp.world) == 0)):
            return self.one_shot.all_reduce(part)      # packets / dense one-shot, or the two-phase form for prefill sizes
        self.comm.all_reduce(part)
        return partial_to_bf16(part)


class ColumnParallel:
    """A column-parallel linear (q/k/v, gate/up): whole activation in, the rank's channels out.  With `gather_cols`
    (an N-split vocabulary head) the ranks' channel blocks are gathered back to the full width on every rank:
    through `one_shot` as one launch over peer memory, else through the process group of `comm`."""

    def __init__(self, linear, comm: Optional[TpCommunicator] = None, one_shot: Optional[OneShotAllReduce] = None,
                 gather_cols: Optional[int] = None):
        if gather_cols is not None and comm is None and one_shot is None:
            raise ValueError("gather_cols needs a communicator")
        self.linear = linear
        self.comm = comm
        self.one_shot = one_shot
        self.gather_cols = gather_cols

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, workspace=None) -> torch.Tensor:
        if self.gather_cols is None:
            return self.linear.forward(x, out=out, workspace=workspace)
        local = self.linear.forward(x, workspace=workspace)
        local = local.reshape(-1, local.shape[-1])
        if self.one_shot is not None and local.numel() <= 2 * min(self.one_shot.max_elems, 524288):
            return self.one_shot.all_gather_cols(local, self.gather_cols, out=out)
        full = self.comm.all_gather_cols(local, self.gather_cols)
        if out is not None:
            out.copy_(full)
            return out
        return full
