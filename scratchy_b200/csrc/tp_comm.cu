// Tensor-parallel exchange for decode: a one-shot all-reduce over NVLink peer memory.
//
// A row-parallel linear (o, down) leaves every rank with f32 partial sums [M, N]; the reference's
// meaning of the collective that follows is "sum the ranks' operands in rank order"
// (crates/compiler/subtile/src/tensor_parallel.rs:1350-1362), then round once.  For the few tokens of
// a decode step the exchange is latency, not bandwidth: one kernel per rank
//   1. stores its partials into a receive slot it owns in EVERY rank's buffer (plain peer stores), each value
//      as an 8-byte packet {f32 bits, call number} — an aligned 8-byte store is single-copy atomic, so the
//      call number doubles as the "value has arrived" flag and neither side needs a system-scope fence
//      (measured: a fence.sys per side cost ~3 us each, twice the rest of the exchange),
//   2. reads — bounded polls — every rank's packets for the elements it owns,
//   3. sums the W received copies in rank order 0..W-1 and rounds to bf16.
// The result is the rank-ordered sum bit for bit on every rank (a library all-reduce promises no
// order).  Buffers are cudaMalloc'd per rank and mapped into the peers through CUDA IPC handles that
// the host exchanges once at start-up; the step path allocates nothing.  No multicast, no TMA here:
// peer memory is only ever touched by ordinary loads and stores of this kernel.
//
// Calls alternate between two halves of the receive area (by a device-side call counter), which is
// enough: a rank can start call e+1 only after every rank has pushed for call e, i.e. after every rank
// has finished reading call e-1.  The call counter lives on the device and is advanced by the last CTA
// of a launch, so a captured CUDA graph replays correctly.
#include "tp_comm.cuh"

#include <string.h>

#include <algorithm>
#include <new>

namespace {

__global__ void __launch_bounds__(TPC_THREADS) tp_allreduce_kernel(TpcPeers peers, int world, int rank, long long max_elems,
                                                                   const float* __restrict__ partial, long long count,
                                                                   uint16_t* __restrict__ y_bf16, float* __restrict__ y_f32,
                                                                   unsigned int* state, int* status, unsigned int wait_limit) {
    __shared__ unsigned int s_epoch;
    const int c = blockIdx.x, tid = threadIdx.x;
    // Programmatic dependent launch: the next kernel of the stream (a matvec that prefetches its load-time
    // weights before its own dependency wait) may start while this exchange is in flight; this kernel itself
    // touches nothing before the kernels ahead of it have completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(&state[0]) + 1u;
    __syncthreads();
    const unsigned int e = s_epoch;

    // 1. my partials, as packets, -> my slot in every rank's receive area
    for (long long base = (long long)c * TPC_SLICE; base < count; base += (long long)gridDim.x * TPC_SLICE) {
        const long long i = base + tid * 4;
        if (i < count) {
            const float4 v = *reinterpret_cast<const float4*>(partial + i);
            const float f[4] = {v.x, v.y, v.z, v.w};
            for (int p = 0; p < world; ++p) {
                uint2* dst = peers.ll[p] + tpc_slot(e, world, rank, max_elems, i);
#pragma unroll
                for (int k = 0; k < 4; ++k) tpc_ll_store(dst + k, f[k], e);
            }
        }
    }
    // 2. every rank's packets for my elements (bounded waits), summed in rank order, one rounding
    const uint2* mine = peers.ll[rank];
    for (long long base = (long long)c * TPC_SLICE; base < count; base += (long long)gridDim.x * TPC_SLICE) {
        const long long i = base + tid * 4;
        if (i < count) {
            float s[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] = tpc_ll_wait(mine + tpc_slot(e, world, 0, max_elems, i) + k, e, status, wait_limit);
            for (int q = 1; q < world; ++q) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    s[k] = __fadd_rn(s[k], tpc_ll_wait(mine + tpc_slot(e, world, q, max_elems, i) + k, e, status, wait_limit));
            }
            if (y_f32) *reinterpret_cast<float4*>(y_f32 + i) = make_float4(s[0], s[1], s[2], s[3]);
            if (y_bf16) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(s[0], s[1]), hi = __floats2bfloat162_rn(s[2], s[3]);
                *reinterpret_cast<uint2*>(y_bf16 + i) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            }
        }
    }
    // 3. the last CTA to finish advances the call counter (every CTA has read it by then)
    tpc_finish_call(state, e, gridDim.x);
}

// The same exchange for larger payloads: dense f32 stores, then one flag per CTA and rank.
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(TPC_THREADS) tp_allreduce_flags_kernel(TpcPeers peers, int world, int rank, long long max_elems,
                                                                         const float* __restrict__ partial, long long count,
                                                                         uint16_t* __restrict__ y_bf16, float* __restrict__ y_f32,
                                                                         unsigned int* state, int* status, unsigned int wait_limit) {
    __shared__ unsigned int s_epoch;
    const int c = blockIdx.x, tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(&state[0]) + 1u;
    __syncthreads();
    const unsigned int e = s_epoch;
    const long long half = (long long)(e & 1u) * world;

    // 1. my partials -> my slot in every rank's dense receive area
    for (long long base = (long long)c * TPC_SLICE; base < count; base += (long long)gridDim.x * TPC_SLICE) {
        const long long i = base + tid * 4;
        if (i < count) {
            const float4 v = *reinterpret_cast<const float4*>(partial + i);
            for (int p = 0; p < world; ++p) *reinterpret_cast<float4*>(peers.recv[p] + (half + rank) * max_elems + i) = v;
        }
    }
    __syncthreads();
    // 2. publish (the release is cumulative over the stores the barrier ordered before it: one system-scope fence
    //    per publishing thread, not one per storing thread), 3. wait for every rank's copy of my slices (bounded)
    if (tid < world) {
        tpc_st_release_sys(peers.flags[tid] + (half + rank) * TPC_MAX_CTAS + c, e);
        const unsigned int* mine = peers.flags[rank] + (half + tid) * TPC_MAX_CTAS + c;
        bool seen = false;
        for (unsigned int it = 0; it < wait_limit; ++it) {
            if ((int)(tpc_ld_acquire_sys(mine) - e) >= 0) {
                seen = true;
                break;
            }
            if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) break;
        }
        if (!seen) atomicCAS(status, 0, TPC_ERR_FLAG_WAIT);
    }
    __syncthreads();
    // 4. rank-ordered sum, one rounding
    const float* mine_recv = peers.recv[rank];
    for (long long base = (long long)c * TPC_SLICE; base < count; base += (long long)gridDim.x * TPC_SLICE) {
        const long long i = base + tid * 4;
        if (i < count) {
            float4 s = ld_cg_f4(mine_recv + half * max_elems + i);
            for (int q = 1; q < world; ++q) {
                const float4 v = ld_cg_f4(mine_recv + (half + q) * max_elems + i);
                s.x = __fadd_rn(s.x, v.x);
                s.y = __fadd_rn(s.y, v.y);
                s.z = __fadd_rn(s.z, v.z);
                s.w = __fadd_rn(s.w, v.w);
            }
            if (y_f32) *reinterpret_cast<float4*>(y_f32 + i) = s;
            if (y_bf16) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
                *reinterpret_cast<uint2*>(y_bf16 + i) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            }
        }
    }
    tpc_finish_call(state, e, gridDim.x);
}

// ---- two phases in one kernel, for prefill-size payloads (count a multiple of 8 * world) --------------------
// CTA c of every rank owns the same sub-range of every slice, so the flags CTA c exchanges with the peers' CTA c
// cover exactly the data it reads.
__device__ __forceinline__ void tpc_flag_round(unsigned int* const* flags2, int phase, long long half, int world, int rank, int c,
                                               unsigned int e, int* status, unsigned int wait_limit) {
    __syncthreads();                                    // this CTA's stores are ordered before the release below
    const int tid = threadIdx.x;
    if (tid < world) {
        const long long row = ((long long)phase * 2 + half) * world;
        tpc_st_release_sys(flags2[tid] + (row + rank) * TPC_MAX_CTAS + c, e);
        const unsigned int* mine = flags2[rank] + (row + tid) * TPC_MAX_CTAS + c;
        bool seen = false;
        for (unsigned int it = 0; it < wait_limit; ++it) {
            if ((int)(tpc_ld_acquire_sys(mine) - e) >= 0) {
                seen = true;
                break;
            }
            if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) break;
        }
        if (!seen) atomicCAS(status, 0, TPC_ERR_FLAG_WAIT);
    }
    __syncthreads();
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(TPC_THREADS) tp_allreduce_two_phase_kernel(TpcPeers peers, int world, int rank, long long ag_stride,
                                                                             long long slice_max, const float* __restrict__ partial,
                                                                             long long count, uint16_t* __restrict__ y_bf16,
                                                                             unsigned int* state, int* status, unsigned int wait_limit) {
    __shared__ unsigned int s_epoch;
    const int c = blockIdx.x, tid = threadIdx.x, G = gridDim.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(&state[0]) + 1u;
    __syncthreads();
    const unsigned int e = s_epoch;
    const long long half = (long long)(e & 1u);
    const long long S = count / world;                   // elements per slice (a multiple of 8)
    const long long per = ((S / 8 + G - 1) / G) * 8;     // this CTA's sub-range of a slice
    const long long lo = (long long)c * per, hi = min(S, lo + per);

    // 1. reduce-scatter, pushed: slice q of my partials -> my row of rank q's receive area (starting with my right
    //    neighbour, so that at any moment the ranks write to different peers)
    for (int dq = 0; dq < world; ++dq) {
        const int q = (rank + 1 + dq) % world;
        const float* src = partial + q * S;
        float* dst = peers.rs[q] + (half * world + rank) * slice_max;
        for (long long i = lo + tid * 4; i < hi; i += TPC_THREADS * 4) *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
    }
    tpc_flag_round(peers.flags2, 0, half, world, rank, c, e, status, wait_limit);

    // 2. my slice: the W copies summed in rank order, one rounding, the bf16 values pushed to every rank (all-gather)
    const float* mine = peers.rs[rank] + half * world * slice_max;
    for (long long i = lo + tid * 8; i < hi; i += TPC_THREADS * 8) {
        float4 a = ld_cg_f4(mine + i), b = ld_cg_f4(mine + i + 4);
        for (int p = 1; p < world; ++p) {
            const float4 u = ld_cg_f4(mine + p * slice_max + i), v = ld_cg_f4(mine + p * slice_max + i + 4);
            a.x = __fadd_rn(a.x, u.x); a.y = __fadd_rn(a.y, u.y); a.z = __fadd_rn(a.z, u.z); a.w = __fadd_rn(a.w, u.w);
            b.x = __fadd_rn(b.x, v.x); b.y = __fadd_rn(b.y, v.y); b.z = __fadd_rn(b.z, v.z); b.w = __fadd_rn(b.w, v.w);
        }
        const __nv_bfloat162 r0 = __floats2bfloat162_rn(a.x, a.y), r1 = __floats2bfloat162_rn(a.z, a.w);
        const __nv_bfloat162 r2 = __floats2bfloat162_rn(b.x, b.y), r3 = __floats2bfloat162_rn(b.z, b.w);
        const uint4 o = make_uint4(*reinterpret_cast<const uint32_t*>(&r0), *reinterpret_cast<const uint32_t*>(&r1),
                                   *reinterpret_cast<const uint32_t*>(&r2), *reinterpret_cast<const uint32_t*>(&r3));
        for (int dq = 0; dq < world; ++dq) {
            const int q = (rank + 1 + dq) % world;
            *reinterpret_cast<uint4*>(peers.ag[q] + half * ag_stride + rank * S + i) = o;
        }
    }
    tpc_flag_round(peers.flags2, 1, half, world, rank, c, e, status, wait_limit);

    // 3. everybody's slices have arrived here: into the caller's output
    const uint16_t* got = peers.ag[rank] + half * ag_stride;
    for (int q = 0; q < world; ++q)
        for (long long i = lo + tid * 8; i < hi; i += TPC_THREADS * 8)
            *reinterpret_cast<uint4*>(y_bf16 + q * S + i) = ld_cg_u4(got + q * S + i);
    tpc_finish_call(state, e, gridDim.x);
}

// ---- all-gather of column blocks (the reference's `SubOp::AllGather{cols}`: an N-split projection, e.g. the
// vocabulary head, restores its full width; crates/compiler/subtile/src/tensor_parallel.rs:1363-1386) -----------
// Every rank holds `rows` x `lc` bf16 values; the result on every rank is, row by row, the ranks' blocks in
// absolute rank order, cropped to `cols` (a padded last block's tail is cut off).  Each CTA pushes its sub-range of
// the local block into this rank's row of every rank's dense receive area (16-byte peer stores), publishes one flag
// per rank, waits (bounded) for the peers' CTA of the same index, and copies that sub-range of every rank's block
// into place.  VEC: lc is a multiple of 8, so a 16-byte chunk never straddles a row.
template <bool VEC>
__global__ void __launch_bounds__(TPC_THREADS) tp_allgather_cols_kernel(TpcPeers peers, int world, int rank, long long one_elems,
                                                                        const uint16_t* __restrict__ local, long long rows, long long lc,
                                                                        long long cols, uint16_t* __restrict__ y, unsigned int* state,
                                                                        int* status, unsigned int wait_limit) {
    __shared__ unsigned int s_epoch;
    const int c = blockIdx.x, tid = threadIdx.x, G = gridDim.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(&state[0]) + 1u;
    __syncthreads();
    const unsigned int e = s_epoch;
    const long long half = (long long)(e & 1u) * world;
    const long long n = rows * lc;                           // bf16 values of one block
    const long long slot = 2 * one_elems;                    // bf16 values one (half, rank) row of the dense area holds
    const long long per = (((n + 7) / 8 + G - 1) / G) * 8;   // this CTA's sub-range, in whole 16-byte chunks
    const long long lo = (long long)c * per, hi = min(n, lo + per);

    // 1. my block -> my row of every rank's receive area
    if (VEC) {
        for (long long i = lo + tid * 8; i < hi; i += TPC_THREADS * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(local + i);
            for (int dq = 0; dq < world; ++dq) {
                const int q = (rank + 1 + dq) % world;
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(peers.recv[q]) + (half + rank) * slot + i) = v;
            }
        }
    } else {
        for (long long i = lo + tid; i < hi; i += TPC_THREADS) {
            const uint16_t v = local[i];
            for (int q = 0; q < world; ++q) (reinterpret_cast<uint16_t*>(peers.recv[q]) + (half + rank) * slot)[i] = v;
        }
    }
    __syncthreads();
    // 2. publish, 3. wait for every rank's CTA c (bounded)
    if (tid < world) {
        tpc_st_release_sys(peers.flags[tid] + (half + rank) * TPC_MAX_CTAS + c, e);
        const unsigned int* mine = peers.flags[rank] + (half + tid) * TPC_MAX_CTAS + c;
        bool seen = false;
        for (unsigned int it = 0; it < wait_limit; ++it) {
            if ((int)(tpc_ld_acquire_sys(mine) - e) >= 0) {
                seen = true;
                break;
            }
            if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) break;
        }
        if (!seen) atomicCAS(status, 0, TPC_ERR_FLAG_WAIT);
    }
    __syncthreads();
    // 4. the blocks into place, rank order along the columns, cropped to `cols`
    const uint16_t* got = reinterpret_cast<const uint16_t*>(peers.recv[rank]) + half * slot;
    for (int q = 0; q < world; ++q) {
        const uint16_t* blk = got + q * slot;
        if (VEC) {
            for (long long i = lo + tid * 8; i < hi; i += TPC_THREADS * 8) {
                const long long row = i / lc, col = q * lc + (i - row * lc);
                if (col >= cols) continue;
                const uint4 v = ld_cg_u4(blk + i);
                uint16_t* dst = y + row * cols + col;
                if (col + 8 <= cols && ((row * cols + col) & 7) == 0) {
                    *reinterpret_cast<uint4*>(dst) = v;
                } else {
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                    for (int j = 0; j < 8 && col + j < cols; ++j) dst[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
                }
            }
        } else {
            for (long long i = lo + tid; i < hi; i += TPC_THREADS) {
                const long long row = i / lc, col = q * lc + (i - row * lc);
                if (col < cols) y[row * cols + col] = *reinterpret_cast<const volatile uint16_t*>(blk + i);
            }
        }
    }
    tpc_finish_call(state, e, gridDim.x);
}

}  // namespace

extern "C" int32_t scr_tp_comm_create(scr_ctx* ctx, int32_t world, int32_t rank, int64_t max_elems, scr_tp_comm** out,
                                      uint8_t* handle_out) {
    SCR_REQUIRE_CTX(ctx);
    if (!out || !handle_out) return scr_fail(ctx, SCR_E_ARG, "tp comm: null pointer");
    *out = nullptr;
    if (!(world == 1 || world == 2 || world == 4 || world == 8) || rank < 0 || rank >= world)
        return scr_fail(ctx, SCR_E_ARG, "tp comm: world %d / rank %d (worlds 1, 2, 4, 8)", world, rank);
    if (max_elems <= 0 || max_elems % 4 != 0) return scr_fail(ctx, SCR_E_SHAPE, "tp comm: max_elems must be a positive multiple of 4");
    static_assert(sizeof(cudaIpcMemHandle_t) == SCR_TP_HANDLE_BYTES, "IPC handle size");
    scr_tp_comm* c = new (std::nothrow) scr_tp_comm();
    if (!c) return scr_fail(ctx, SCR_E_CUDA, "tp comm: out of host memory");
    c->ctx = ctx;
    c->world = world;
    c->rank = rank;
    c->max_elems = max_elems;
    c->one_elems = std::min<long long>(max_elems, TPC_ONE_SHOT_MAX);
    c->slice_max = ((max_elems + world - 1) / world + 7) / 8 * 8;
    // one-shot: packets | dense f32 | flags; two-phase: received slices | gathered result | flags.  Zeroed: call numbers start at 1
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    c->recv_off = up((size_t)2 * world * c->one_elems * sizeof(uint2));
    c->flags_off = up(c->recv_off + (size_t)2 * world * c->one_elems * sizeof(float));
    c->rs_off = up(c->flags_off + (size_t)2 * world * TPC_MAX_CTAS * sizeof(unsigned int));
    c->bytes = c->rs_off;
    if (max_elems >= TPC_TWO_PHASE_MIN) {
        c->ag_off = up(c->rs_off + (size_t)2 * world * c->slice_max * sizeof(float));
        c->flags2_off = up(c->ag_off + (size_t)2 * ((max_elems + 7) / 8 * 8) * sizeof(uint16_t));
        c->bytes = c->flags2_off + (size_t)2 * 2 * world * TPC_MAX_CTAS * sizeof(unsigned int);
    }
    cudaError_t e = cudaMalloc((void**)&c->local, c->bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, c->bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->state, 2 * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(c->state, 0, 2 * sizeof(unsigned int));
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, c->local);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (c->local) cudaFree(c->local);
        if (c->state) cudaFree(c->state);
        delete c;
        return scr_fail(ctx, SCR_E_CUDA, "tp comm: %s", cudaGetErrorString(e));
    }
    memcpy(handle_out, &h, sizeof(h));
    c->peer[rank] = c->local;
    c->connected = (world == 1);
    *out = c;
    return SCR_OK;
}

extern "C" int32_t scr_tp_comm_connect(scr_tp_comm* comm, const uint8_t* handles) {
    if (!comm || !handles) return SCR_E_ARG;
    scr_ctx* ctx = comm->ctx;
    for (int p = 0; p < comm->world; ++p) {
        if (p == comm->rank || comm->opened[p]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)p * SCR_TP_HANDLE_BYTES, sizeof(h));
        void* ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return scr_fail(ctx, SCR_E_COMM, "tp comm: cannot map rank %d's buffer: %s", p, cudaGetErrorString(e));
        comm->peer[p] = static_cast<unsigned char*>(ptr);
        comm->opened[p] = true;
    }
    comm->connected = true;
    return SCR_OK;
}

// Ranks that are threads of ONE process (the reference's executor runs one OS thread per rank inside one process:
// crates/serving/worker/src/threadpool.rs:1-16, parallel.rs:103-150) cannot open each other's IPC handles — an IPC
// handle only opens in another process.  They connect with raw device pointers instead: every rank publishes
// `scr_tp_comm_base`, and each calls this with all W bases and the devices they live on, with its own device
// current.  Peer access is enabled here (an already-enabled pair is fine).
extern "C" int32_t scr_tp_comm_base(scr_tp_comm* comm, void** base) {
    if (!comm || !base) return SCR_E_ARG;
    *base = comm->local;
    return SCR_OK;
}

extern "C" int32_t scr_tp_comm_connect_local(scr_tp_comm* comm, void* const* peer_bases, const int32_t* peer_devices) {
    if (!comm || !peer_bases || !peer_devices) return SCR_E_ARG;
    scr_ctx* ctx = comm->ctx;
    SCR_REQUIRE_CTX(ctx);
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device)
        return scr_fail(ctx, SCR_E_ARG, "tp comm: device %d must be current (current is %d)", ctx->device, cur);
    for (int p = 0; p < comm->world; ++p) {
        if (p == comm->rank) continue;
        if (!peer_bases[p]) return scr_fail(ctx, SCR_E_ARG, "tp comm: rank %d has no base pointer", p);
        if (peer_devices[p] != ctx->device) {
            int can = 0;
            cudaError_t e = cudaDeviceCanAccessPeer(&can, ctx->device, peer_devices[p]);
            if (e != cudaSuccess || !can)
                return scr_fail(ctx, SCR_E_COMM, "tp comm: device %d cannot reach device %d", ctx->device, peer_devices[p]);
            e = cudaDeviceEnablePeerAccess(peer_devices[p], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) {
                (void)cudaGetLastError();
            } else if (e != cudaSuccess) {
                return scr_fail(ctx, SCR_E_COMM, "tp comm: enabling peer access to device %d: %s", peer_devices[p], cudaGetErrorString(e));
            }
        }
        comm->peer[p] = static_cast<unsigned char*>(peer_bases[p]);
    }
    comm->connected = true;
    return SCR_OK;
}

// How many times a kernel polls for a peer's packet or flag before it gives up, records SCR_E_TIMEOUT's code in the
// context's status word and runs to its end (results of that call are garbage; the call counter still advances, so
// the next call works).  The default is generous; health checks and tests set it short.
extern "C" int32_t scr_tp_comm_set_wait_limit(scr_tp_comm* comm, uint32_t polls) {
    if (!comm || polls == 0) return SCR_E_ARG;
    comm->wait_limit = polls;
    return SCR_OK;
}

extern "C" int32_t scr_tp_allreduce_partial(scr_tp_comm* comm, const float* partial, int64_t count, uint16_t* y_bf16,
                                            float* y_f32, void* stream) {
    if (!comm) return SCR_E_ARG;
    scr_ctx* ctx = comm->ctx;
    SCR_REQUIRE_CTX(ctx);
    if (!partial || (!y_bf16 && !y_f32)) return scr_fail(ctx, SCR_E_ARG, "tp all-reduce: null pointer");
    if (!comm->connected) return scr_fail(ctx, SCR_E_COMM, "tp all-reduce: peers are not connected");
    if (count <= 0 || count % 4 != 0 || count > comm->max_elems)
        return scr_fail(ctx, SCR_E_SHAPE, "tp all-reduce: count %lld must be a positive multiple of 4, at most %lld", (long long)count,
                        comm->max_elems);
    if (!scr_aligned16(partial) || (y_f32 && !scr_aligned16(y_f32)) || (y_bf16 && ((uintptr_t)y_bf16 & 7u)))
        return scr_fail(ctx, SCR_E_ALIGN, "tp all-reduce: buffers must be 16-byte aligned");
    const TpcPeers peers = tpc_peer_table(comm);
    const bool two_phase = count >= TPC_TWO_PHASE_MIN && count % (8 * comm->world) == 0 && y_bf16 && !y_f32 &&
                           comm->max_elems >= TPC_TWO_PHASE_MIN && scr_aligned16(y_bf16);
    if (!two_phase && count > comm->one_elems)
        return scr_fail(ctx, SCR_E_SHAPE, "tp all-reduce: %lld values need the two-phase form (bf16 output only, count a multiple of %d)",
                        (long long)count, 8 * comm->world);
    const int grid = two_phase ? std::min(ctx->sm_count, TPC_MAX_CTAS)
                               : (int)std::min<long long>((count + TPC_SLICE - 1) / TPC_SLICE, TPC_MAX_GRID);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TPC_THREADS);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // every rank takes the same branch: count, world and the output kinds are the same everywhere
    cudaError_t e;
    if (two_phase) {
        e = cudaLaunchKernelEx(&cfg, tp_allreduce_two_phase_kernel, peers, comm->world, comm->rank, (long long)((comm->max_elems + 7) / 8 * 8),
                               (long long)comm->slice_max, partial, (long long)count, y_bf16, comm->state, ctx->dev_status,
                               comm->wait_limit);
    } else {
        auto kernel = (long long)count * comm->world <= TPC_PACKET_MAX ? tp_allreduce_kernel : tp_allreduce_flags_kernel;
        e = cudaLaunchKernelEx(&cfg, kernel, peers, comm->world, comm->rank, (long long)comm->one_elems, partial, (long long)count,
                               y_bf16, y_f32, comm->state, ctx->dev_status, comm->wait_limit);
    }
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "tp all-reduce launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "tp_allreduce");
}

// `SubOp::AllGather{cols}` over peer memory: y[rows, cols] = the ranks' [rows, lc] bf16 column blocks side by side in
// absolute rank order, cropped to `cols` (world * lc >= cols).  One launch; the same bytes on every rank.
extern "C" int32_t scr_tp_allgather_cols(scr_tp_comm* comm, const uint16_t* local_bf16, int64_t rows, int64_t lc, int64_t cols,
                                         uint16_t* y_bf16, void* stream) {
    if (!comm) return SCR_E_ARG;
    scr_ctx* ctx = comm->ctx;
    SCR_REQUIRE_CTX(ctx);
    if (!local_bf16 || !y_bf16) return scr_fail(ctx, SCR_E_ARG, "tp all-gather: null pointer");
    if (!comm->connected) return scr_fail(ctx, SCR_E_COMM, "tp all-gather: peers are not connected");
    if (rows <= 0 || lc <= 0 || cols <= 0) return scr_fail(ctx, SCR_E_SHAPE, "tp all-gather: rows=%lld lc=%lld cols=%lld must be positive",
                                                           (long long)rows, (long long)lc, (long long)cols);
    if (lc * comm->world < cols)
        return scr_fail(ctx, SCR_E_SHAPE, "tp all-gather: %d blocks of %lld columns cannot restore %lld", comm->world, (long long)lc,
                        (long long)cols);
    const long long n = (long long)rows * lc;
    if ((n + 7) / 8 * 8 > 2 * comm->one_elems)
        return scr_fail(ctx, SCR_E_SHAPE, "tp all-gather: a block of %lld values exceeds the receive area (%lld)", n, 2 * comm->one_elems);
    const bool vec = lc % 8 == 0 && scr_aligned16(local_bf16);
    const TpcPeers peers = tpc_peer_table(comm);
    // the same grid on every rank: it depends on the block's size only
    const int grid = (int)std::min<long long>((n + TPC_THREADS * 8 - 1) / (TPC_THREADS * 8), TPC_MAX_GRID);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TPC_THREADS);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto kernel = vec ? tp_allgather_cols_kernel<true> : tp_allgather_cols_kernel<false>;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, peers, comm->world, comm->rank, (long long)comm->one_elems, local_bf16,
                                             (long long)rows, (long long)lc, (long long)cols, y_bf16, comm->state, ctx->dev_status,
                                             comm->wait_limit);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "tp all-gather launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "tp_allgather_cols");
}

extern "C" int32_t scr_tp_comm_destroy(scr_tp_comm* comm) {
    if (!comm) return SCR_E_ARG;
    cudaDeviceSynchronize();
    for (int p = 0; p < comm->world; ++p)
        if (comm->opened[p]) cudaIpcCloseMemHandle(comm->peer[p]);
    if (comm->local) cudaFree(comm->local);
    if (comm->state) cudaFree(comm->state);
    delete comm;
    return SCR_OK;
}
