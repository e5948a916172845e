// The operators either side of the quantized linears in one decode step: embedding gather,
// RMSNorm (plain and fused with the residual add), SiLU(gate)*up, RoPE + paged-KV append,
// paged decode attention and greedy argmax.  bf16 activations, f32 arithmetic.
//
// All of them are byte movers bounded by HBM / launch latency, not by arithmetic: the kernels
// are plain vectorised loads and stores.  The attention kernel splits the KV range of one
// (sequence, kv head) over the 8 CTAs of a thread-block cluster and merges the partial
// softmax states through distributed shared memory, so it needs no workspace and no second
// launch.
//
// Contracts (paths relative to the reference project's root): crates/targets/metal/src/
// cpu_golden.rs:25-37 (rmsnorm), :114-124 (embed), :171-200 (fused_add_rmsnorm), :211-219
// (fused_gate_up_silu_mul), :289-362 (rope_append), :386-460 (attention_via_cache); cache
// addressing crates/targets/metal/src/paged_kv_layout.rs:74-115; argmax tie rule
// crates/targets/metal/tests/argmax_split_test.rs:24-33.
#include "tc_common.cuh"

#include <math.h>

namespace {

// Device-side argument checks record one of these in the context's status word and skip the
// offending access instead of faulting.
constexpr int DEV_BAD_TOKEN_ID = 0x0E000001;
constexpr int DEV_BAD_SLOT = 0x0E000002;
constexpr int DEV_BAD_BLOCK = 0x0E000003;
constexpr int DEV_BAD_POSITION = 0x0E000004;

// Programmatic dependent launch: every kernel here lets the next kernel of the stream start its own
// prologue at once (a following matvec prefetches weights while this kernel runs) and waits for the
// previous kernel's results before it touches any activation.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    const __nv_bfloat16 v = __float2bfloat16_rn(f);
    return uint32_t(*reinterpret_cast<const uint16_t*>(&v));
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xFFFF0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xFFFF0000u);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 v;
    v.x = f32_to_bf16_bits(f[0]) | (f32_to_bf16_bits(f[1]) << 16);
    v.y = f32_to_bf16_bits(f[2]) | (f32_to_bf16_bits(f[3]) << 16);
    v.z = f32_to_bf16_bits(f[4]) | (f32_to_bf16_bits(f[5]) << 16);
    v.w = f32_to_bf16_bits(f[6]) | (f32_to_bf16_bits(f[7]) << 16);
    return v;
}

// ------------------------------------------------------------------------------- embed
__global__ void embed_kernel(const uint32_t* __restrict__ ids, const uint4* __restrict__ table, uint32_t vocab, int hidden_v,
                             uint4* __restrict__ out, int* status) {
    pdl_trigger();
    pdl_wait();
    const uint32_t id = ids[blockIdx.x];
    const bool ok = id < vocab;
    if (!ok && threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_TOKEN_ID);
    const uint4* src = table + size_t(ok ? id : 0) * hidden_v;
    uint4* dst = out + size_t(blockIdx.x) * hidden_v;
    for (int v = threadIdx.x; v < hidden_v; v += blockDim.x) dst[v] = ok ? src[v] : make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------- rmsnorm
constexpr int NORM_THREADS = 256;

__device__ __forceinline__ float norm_block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < NORM_THREADS / 32; ++w) t += red[w];
    return t;
}

// One CTA per row.  ADD: residual <- bf16(residual + delta) in place, and the norm is taken
// off the stored (rounded) residual; out may alias delta.  !ADD: out = rmsnorm(residual).
template <bool ADD>
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_kernel(uint16_t* __restrict__ residual, const uint16_t* delta,
                                                               const uint16_t* __restrict__ weight, uint16_t* out, int hidden,
                                                               float eps) {
    extern __shared__ float row[];          // hidden floats
    __shared__ float red[NORM_THREADS / 32];
    pdl_trigger();
    const int nv = hidden >> 3;
    // the gains are load-time constants (cold in HBM once per step): fetch this thread's share before the
    // wait, so that their latency hides under the previous kernel instead of following the reduction
    constexpr int GAIN_PREFETCH = 4;        // covers hidden <= 8192; beyond that the rest is loaded late
    uint4 gain[GAIN_PREFETCH];
#pragma unroll
    for (int i = 0; i < GAIN_PREFETCH; ++i) {
        const int v = threadIdx.x + i * NORM_THREADS;
        gain[i] = v < nv ? ld_nc_v4(weight + v * 8) : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    const size_t base = size_t(blockIdx.x) * hidden;
    float sum_sq = 0.0f;
    for (int v = threadIdx.x; v < nv; v += NORM_THREADS) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(residual + base + v * 8), f);
        if (ADD) {
            float d[8];
            unpack8(*reinterpret_cast<const uint4*>(delta + base + v * 8), d);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = bf16_bits_to_f32(f32_to_bf16_bits(__fadd_rn(f[j], d[j])));
            *reinterpret_cast<uint4*>(residual + base + v * 8) = pack8(f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            row[v * 8 + j] = f[j];
            sum_sq = __fadd_rn(sum_sq, __fmul_rn(f[j], f[j]));
        }
    }
    const float total = norm_block_sum(sum_sq, red);
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(hidden)), eps));
    const float inv_rms = __fdiv_rn(1.0f, rms);
    for (int v = threadIdx.x, i = 0; v < nv; v += NORM_THREADS, ++i) {
        float w[8], o[8];
        uint4 gv = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < GAIN_PREFETCH; ++u)
            if (u == i) gv = gain[u];
        if (i >= GAIN_PREFETCH) gv = *reinterpret_cast<const uint4*>(weight + v * 8);
        unpack8(gv, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(__fmul_rn(row[v * 8 + j], inv_rms), w[j]);
        *reinterpret_cast<uint4*>(out + base + v * 8) = pack8(o);
    }
}

// ------------------------------------------------------------------------------- silu(gate) * up
// `vstride` = 8 for gate and up as two dense halves, 16 when the fused output interleaves them in runs of 8
// columns (8 gate, then the 8 up of the same channels: the layout of the matvec's pairing epilogue).
__global__ void silu_mul_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up, long long ld_in,
                                uint16_t* __restrict__ out, int inter_v, long long total_v, int vstride) {
    pdl_trigger();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_v; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / inter_v;
        const int v = int(i - r * inter_v);
        float g[8], u[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(gate + r * ld_in + v * vstride), g);
        unpack8(*reinterpret_cast<const uint4*>(up + r * ld_in + v * vstride), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(__fdiv_rn(g[j], __fadd_rn(1.0f, expf(-g[j]))), u[j]);
        *reinterpret_cast<uint4*>(out + (r * inter_v + v) * 8) = pack8(o);
    }
}

// ------------------------------------------------------------------------------- rope + append
// grid (num_q_heads + num_kv_heads, tokens).  A q-head CTA writes the rotated q; a kv-head
// CTA writes the rotated k and the unrotated v into the token's cache slot.  Products and
// the sum/difference are rounded separately (no fused multiply-add), as the contract's f32
// statement does, so the stored bf16 values are exactly the rounded reference values.
__global__ void rope_append_kernel(const uint16_t* q, long long ld_q, const uint16_t* __restrict__ k, long long ld_k,
                                   const uint16_t* __restrict__ v, long long ld_v, const uint32_t* __restrict__ positions,
                                   const uint32_t* __restrict__ slot_mapping, const float* __restrict__ cos_table,
                                   const float* __restrict__ sin_table, uint32_t max_pos, uint16_t* q_out,
                                   long long ld_qo, uint16_t* __restrict__ cache_k, uint16_t* __restrict__ cache_v,
                                   uint32_t num_blocks, int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                   int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    const int h = blockIdx.x;
    const int half = head_dim >> 1;
    const uint32_t pos = positions[t];
    if (pos >= max_pos) {
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_POSITION);
        return;
    }
    const float* cos_row = cos_table + size_t(pos) * head_dim;
    const float* sin_row = sin_table + size_t(pos) * head_dim;
    if (h < num_q_heads) {
        const uint16_t* src = q + t * ld_q + h * head_dim;
        uint16_t* dst = q_out + t * ld_qo + h * head_dim;
        for (int d = threadIdx.x; d < half; d += blockDim.x) {
            const float x0 = bf16_bits_to_f32(src[d]), x1 = bf16_bits_to_f32(src[half + d]);
            const float c = cos_row[d], s = sin_row[d];
            const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            const float r1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
            dst[d] = uint16_t(f32_to_bf16_bits(r0));
            dst[half + d] = uint16_t(f32_to_bf16_bits(r1));
        }
        return;
    }
    const int kh = h - num_q_heads;
    const uint32_t slot = slot_mapping[t];
    const uint32_t block = slot / uint32_t(block_size), in_block = slot % uint32_t(block_size);
    if (block >= num_blocks) {
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_SLOT);
        return;
    }
    const size_t cache_base = ((size_t(block) * num_kv_heads + kh) * block_size + in_block) * head_dim;
    const uint16_t* ksrc = k + t * ld_k + kh * head_dim;
    const uint16_t* vsrc = v + t * ld_v + kh * head_dim;
    for (int d = threadIdx.x; d < half; d += blockDim.x) {
        const float x0 = bf16_bits_to_f32(ksrc[d]), x1 = bf16_bits_to_f32(ksrc[half + d]);
        const float c = cos_row[d], s = sin_row[d];
        const float r0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        const float r1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
        cache_k[cache_base + d] = uint16_t(f32_to_bf16_bits(r0));
        cache_k[cache_base + half + d] = uint16_t(f32_to_bf16_bits(r1));
        cache_v[cache_base + d] = vsrc[d];
        cache_v[cache_base + half + d] = vsrc[half + d];
    }
}

// ------------------------------------------------------------------------------- argmax
// One CTA per row: the largest value, the smallest index among equal ones, NaN never.
constexpr int ARGMAX_THREADS = 1024;

__device__ __forceinline__ void argmax_take(float v, uint32_t i, float& best, uint32_t& best_i) {
    if (v > best || (v == best && i < best_i)) {
        best = v;
        best_i = i;
    }
}

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const uint16_t* __restrict__ logits, long long ld, int width,
                                                                uint32_t* __restrict__ out) {
    __shared__ float s_best[ARGMAX_THREADS / 32];
    __shared__ uint32_t s_idx[ARGMAX_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const uint16_t* row = logits + blockIdx.x * ld;
    float best = -INFINITY;
    uint32_t best_i = 0;
    const int nv = width >> 3;
    for (int v = threadIdx.x; v < nv; v += ARGMAX_THREADS) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(row + v * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) argmax_take(f[j], uint32_t(v * 8 + j), best, best_i);
    }
    for (int i = (nv << 3) + threadIdx.x; i < width; i += ARGMAX_THREADS)
        argmax_take(bf16_bits_to_f32(row[i]), uint32_t(i), best, best_i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        argmax_take(ob, oi, best, best_i);
    }
    if ((threadIdx.x & 31) == 0) {
        s_best[threadIdx.x >> 5] = best;
        s_idx[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < ARGMAX_THREADS / 32; ++w) argmax_take(s_best[w], s_idx[w], best, best_i);
        out[blockIdx.x] = best_i;
    }
}


// ------------------------------------------------------------------------------- paged decode attention
// grid (ATT_SPLITS, num_kv_heads, batch), one cluster of ATT_SPLITS CTAs per (sequence, kv
// head).  CTA `split` streams tokens [split*per, (split+1)*per) of the sequence's KV once and
// serves all G query heads that share the kv head from the same loads.  LPT = D/8 lanes hold
// one token's 16-byte pieces; every lane group keeps an online-softmax state (running maximum
// m, sum l, weighted V sum) per query head.  States are merged lane group -> warp -> CTA ->
// cluster; CTA 0 of the cluster applies inv_sum = 1 / (l + 1e-6) and stores bf16.
constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int ATT_SPLITS = 8;
constexpr uint32_t ATT_NO_BLOCK = 0xFFFFFFFFu;

__device__ __forceinline__ uint32_t att_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void att_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Store `v` at the address of `local` inside CTA 0 of the cluster.
__device__ __forceinline__ void att_store_rank0(float* local, float v) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(a), "r"(0));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ float att_weight(float m, float m_new) { return m == -INFINITY ? 0.0f : expf(m - m_new); }


// Warps -> CTA: called by the ATT_THREADS consumer threads once every warp has written its state
// (acc[D], m, l per query head) to warp_part[warp][g].  With one split the output row is stored
// directly; otherwise the CTA's state goes to CTA 0's table through distributed shared memory.
template <int D>
__device__ __forceinline__ void att_cta_merge(int G, int nwarps, const float* warp_part, float* cl_part, int split, int nsplit,
                                              int q_head0, int b, uint16_t* __restrict__ out, long long ld_o) {
    constexpr int STATE = D + 2;
    __shared__ float wgt[8][ATT_WARPS + 2];          // per query head: the warps' weights, the merged maximum and sum
    const int nthreads = nwarps * 32;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        float mt = -INFINITY;
        for (int w = 0; w < nwarps; ++w) mt = fmaxf(mt, warp_part[(w * G + g) * STATE + D]);
        float lt = 0.0f;
        for (int w = 0; w < nwarps; ++w) {
            const float c = att_weight(warp_part[(w * G + g) * STATE + D], mt);
            wgt[g][w] = c;
            lt += warp_part[(w * G + g) * STATE + D + 1] * c;
        }
        wgt[g][ATT_WARPS] = mt;
        wgt[g][ATT_WARPS + 1] = lt;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    for (int idx = threadIdx.x; idx < G * D; idx += nthreads) {
        const int g = idx / D, d = idx - g * D;
        float a = 0.0f;
        for (int w = 0; w < nwarps; ++w) a += warp_part[(w * G + g) * STATE + d] * wgt[g][w];
        if (nsplit == 1) {
            out[b * ld_o + (q_head0 + g) * D + d] = uint16_t(f32_to_bf16_bits(a * __fdiv_rn(1.0f, wgt[g][ATT_WARPS + 1] + 1e-6f)));
        } else {
            float* dst = cl_part + (split * G + g) * STATE;
            att_store_rank0(dst + d, a);
            if (d == 0) {
                att_store_rank0(dst + D, wgt[g][ATT_WARPS]);
                att_store_rank0(dst + D + 1, wgt[g][ATT_WARPS + 1]);
            }
        }
    }
}

// Merge of the per-lane-group online-softmax states: lane groups -> warp (shuffles) -> CTA
// (shared memory) -> cluster (stores into CTA 0's table through distributed shared memory).
// CTA 0 of the cluster applies inv_sum = 1 / (l + 1e-6) and stores bf16.  Called by all
// threads of the first ATT_THREADS (the consumer warps); `bar_id` names the CTA barrier they share.
template <int D, int G>
__device__ __forceinline__ void att_merge_and_store(float (&m)[G], float (&lsum)[G], float (&acc)[G][8], float* warp_part,
                                                    float* cl_part, int split, int nsplit, int q_head0, int b,
                                                    uint16_t* __restrict__ out, long long ld_o) {
    constexpr int LPT = D / 8;
    constexpr int STATE = D + 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane / LPT, l = lane % LPT;
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
            const float lo = __shfl_xor_sync(0xffffffffu, lsum[g], o);
            const float mn = fmaxf(m[g], mo);
            const float ca = att_weight(m[g], mn), cb = att_weight(mo, mn);
            lsum[g] = lsum[g] * ca + lo * cb;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][j], o);
                acc[g][j] = acc[g][j] * ca + ao * cb;
            }
            m[g] = mn;
        }
    }
    if (grp == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float* st = warp_part + (warp * G + g) * STATE;
#pragma unroll
            for (int j = 0; j < 8; ++j) st[l * 8 + j] = acc[g][j];
            if (l == 0) {
                st[D] = m[g];
                st[D + 1] = lsum[g];
            }
        }
    }
    att_cta_merge<D>(G, ATT_WARPS, warp_part, cl_part, split, nsplit, q_head0, b, out, ld_o);
}

// After the cluster barrier: CTA 0 folds the splits' states and stores the output row.  Called by
// every thread of CTA 0 (`nthreads` of them).
template <int D>
__device__ __forceinline__ void att_cluster_finish(int G, const float* cl_part, int nsplit, int q_head0, int b,
                                                   uint16_t* __restrict__ out, long long ld_o, int nthreads) {
    constexpr int STATE = D + 2;
    __shared__ float swgt[8][ATT_SPLITS + 1];        // per query head: the splits' weights and 1 / (sum + 1e-6)
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        float mt = -INFINITY;
        for (int sp = 0; sp < nsplit; ++sp) mt = fmaxf(mt, cl_part[(sp * G + g) * STATE + D]);
        float lt = 0.0f;
        for (int sp = 0; sp < nsplit; ++sp) {
            const float c = att_weight(cl_part[(sp * G + g) * STATE + D], mt);
            swgt[g][sp] = c;
            lt += cl_part[(sp * G + g) * STATE + D + 1] * c;
        }
        swgt[g][ATT_SPLITS] = __fdiv_rn(1.0f, lt + 1e-6f);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += nthreads) {
        const int g = idx / D, d = idx - g * D;
        float a = 0.0f;
        for (int sp = 0; sp < nsplit; ++sp) a += cl_part[(sp * G + g) * STATE + d] * swgt[g][sp];
        out[b * ld_o + (q_head0 + g) * D + d] = uint16_t(f32_to_bf16_bits(a * swgt[g][ATT_SPLITS]));
    }
}

template <int D, int G>
__global__ void __launch_bounds__(ATT_THREADS) attention_decode_kernel(
    const uint16_t* __restrict__ q, long long ld_q, const uint16_t* __restrict__ cache_k, const uint16_t* __restrict__ cache_v,
    const uint32_t* __restrict__ block_table, const uint32_t* __restrict__ seq_used_k, uint16_t* __restrict__ out, long long ld_o,
    int num_kv_heads, int block_size, int max_blocks_per_seq, uint32_t num_blocks, int table_cap, float scale, int* status) {
    constexpr int LPT = D / 8;
    constexpr int TPW = 32 / LPT;
    constexpr int STATE = D + 2;                     // acc[D], m, l
    constexpr int U = G <= 4 ? 4 : 2;                // tokens in flight per lane group
    extern __shared__ __align__(128) unsigned char att_smem[];
    float* warp_part = reinterpret_cast<float*>(att_smem);                 // [ATT_WARPS][G][STATE]
    float* cl_part = warp_part + ATT_WARPS * G * STATE;                    // [ATT_SPLITS][G][STATE], filled on CTA 0
    uint32_t* blocks = reinterpret_cast<uint32_t*>(cl_part + ATT_SPLITS * G * STATE);

    pdl_trigger();
    pdl_wait();
    const int split = int(att_cluster_rank());
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane / LPT, l = lane % LPT;

    long long kv_len_raw = seq_used_k[b];
    const long long kv_cap = (long long)max_blocks_per_seq * block_size;
    if (kv_len_raw > kv_cap) {
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_BLOCK);
        kv_len_raw = kv_cap;
    }
    const int kv_len = int(kv_len_raw);
    const int per = (kv_len + ATT_SPLITS - 1) / ATT_SPLITS;
    const int t_begin = min(split * per, kv_len), t_end = min(t_begin + per, kv_len);
    const int first_blk = t_begin / block_size;
    int nblk = t_end > t_begin ? (t_end - 1) / block_size - first_blk + 1 : 0;
    if (nblk > table_cap) {                          // cannot happen for a consistent launch; never index past the slice
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_BLOCK);
        nblk = 0;
    }
    for (int i = threadIdx.x; i < nblk; i += ATT_THREADS) {
        uint32_t pb = block_table[size_t(b) * max_blocks_per_seq + first_blk + i];
        if (pb >= num_blocks) {
            atomicCAS(status, 0, DEV_BAD_BLOCK);
            pb = ATT_NO_BLOCK;
        }
        blocks[i] = pb;
    }
    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) unpack8(*reinterpret_cast<const uint4*>(q + b * ld_q + (kvh * G + g) * D + l * 8), qf[g]);
    __syncthreads();

    float m[G], lsum[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        lsum[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = 0.0f;
    }
    constexpr int PASS = ATT_WARPS * TPW;            // tokens one CTA pass covers
    const int t_last = nblk > 0 ? t_end : t_begin;
    for (int base = t_begin; base < t_last; base += PASS * U) {
        uint4 kk[U], vv[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = base + u * PASS + warp * TPW + grp;
            ok[u] = t < t_last;
            kk[u] = make_uint4(0, 0, 0, 0);
            vv[u] = make_uint4(0, 0, 0, 0);
            if (ok[u]) {
                const int lb = t / block_size;
                const uint32_t pb = blocks[lb - first_blk];
                ok[u] = pb != ATT_NO_BLOCK;
                if (ok[u]) {
                    const size_t off = ((size_t(pb) * num_kv_heads + kvh) * block_size + (t - lb * block_size)) * D + l * 8;
                    kk[u] = ld_stream_v4(cache_k + off);
                    vv[u] = ld_stream_v4(cache_v + off);
                }
            }
        }
        float s[U][G];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float kf[8];
            unpack8(kk[u], kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float p = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) p = fmaf(qf[g][j], kf[j], p);
#pragma unroll
                for (int o = LPT / 2; o > 0; o >>= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
                s[u][g] = ok[u] ? p * scale : -INFINITY;
            }
        }
        float vf[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) unpack8(vv[u], vf[u]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < U; ++u) mn = fmaxf(mn, s[u][g]);
            if (mn == -INFINITY) continue;
            const float corr = att_weight(m[g], mn);
            lsum[g] *= corr;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[g][j] *= corr;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float p = ok[u] ? expf(s[u][g] - mn) : 0.0f;
                lsum[g] += p;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(p, vf[u][j], acc[g][j]);
            }
            m[g] = mn;
        }
    }

    att_merge_and_store<D, G>(m, lsum, acc, warp_part, cl_part, split, ATT_SPLITS, kvh * G, b, out, ld_o);
    att_cluster_sync();
    if (split == 0) att_cluster_finish<D>(G, cl_part, ATT_SPLITS, kvh * G, b, out, ld_o, ATT_THREADS);
}


// ---- the streaming variant: TMA tiles + tensor cores -------------------------------------------
// In the paged layout one (block, kv head) is a contiguous run of block_size tokens x D bf16.  A
// producer warp brings those runs (K and V) into a shared-memory ring with one 3-D TMA tile load
// each (tensor map over the cache viewed as [token][D/64][64], 128-byte swizzle), one ring stage
// per cache block, completion counted in bytes on the stage's mbarrier; everything the ring holds
// is in flight at once.  Each of the eight consumer warps takes whole blocks and runs them through
// mma.sync m16n8k16: S = Q K^T with the (up to 8) query heads of the kv head as the rows of the
// 16-row A operand and K read by ldmatrix; an online softmax on the accumulator fragments; O += P V
// with V read by ldmatrix.trans and P split into a bf16 head and a bf16 remainder (two MMAs), so
// the probabilities keep ~16 mantissa bits.  Scores, the softmax state and O stay in f32.
// The cluster (1, 2, 4 or 8 CTAs, chosen by the host from the batch) splits the sequence by whole
// blocks.  Every wait is bounded and reports through the status word.
constexpr int ATTB_THREADS = ATT_THREADS + 32;
constexpr int ATT_ERR_FULL = 0x0A000001;
constexpr int ATT_ERR_EMPTY = 0x0A000002;

__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* tmap, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16) * B(16x8,bf16).  Rows 8..15 of A are zero here (a1 = a3 = 0), so the
// accumulator halves of those rows (z0, z1) stay zero: callers pass a few shared dummies for them.
__device__ __forceinline__ void mma_bf16_16816(float& c0, float& c1, float& z0, float& z1, uint32_t a0, uint32_t a2, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) { return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16); }

// RoPE + append folded into the attention (`enabled`): q, k_new, v_new are the UNrotated outputs of the QKV
// projection; the kernel rotates q in registers, and the CTA that owns the sequence's newest block rotates k_new,
// writes it and v_new into the token's cache slot (for later steps) and patches them into its shared-memory tile
// (for this one).  Products and sums are rounded as in the stand-alone kernel, so q, the cache and the attention
// output are the same bits as `rope_append` followed by the plain attention.
struct AttRope {
    const uint16_t* k_new;
    const uint16_t* v_new;
    const uint32_t* positions;
    const float* cos_table;
    const float* sin_table;
    uint16_t* cache_k;
    uint16_t* cache_v;
    long long ld_k, ld_v;
    uint32_t max_pos;
    int enabled;
};

__device__ __forceinline__ uint32_t att_rope_pair(uint32_t x0w, uint32_t x1w, const float* c, const float* s, bool first) {
    // two adjacent dims: lo/hi halves of the words; `first` selects the output for d (x0*c - x1*s) or d + half (x1*c + x0*s)
    const float x0l = __uint_as_float(x0w << 16), x0h = __uint_as_float(x0w & 0xFFFF0000u);
    const float x1l = __uint_as_float(x1w << 16), x1h = __uint_as_float(x1w & 0xFFFF0000u);
    float rl, rh;
    if (first) {
        rl = __fsub_rn(__fmul_rn(x0l, c[0]), __fmul_rn(x1l, s[0]));
        rh = __fsub_rn(__fmul_rn(x0h, c[1]), __fmul_rn(x1h, s[1]));
    } else {
        rl = __fadd_rn(__fmul_rn(x1l, c[0]), __fmul_rn(x0l, s[0]));
        rh = __fadd_rn(__fmul_rn(x1h, c[1]), __fmul_rn(x0h, s[1]));
    }
    return pack_bf16x2(rl, rh);
}

template <int D>
__global__ void __launch_bounds__(ATTB_THREADS) attention_decode_tc_kernel(
    const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, const uint16_t* __restrict__ q,
    long long ld_q, const uint32_t* __restrict__ block_table, const uint32_t* __restrict__ seq_used_k,
    uint16_t* __restrict__ out, long long ld_o, int G, int num_kv_heads, int block_size, int max_blocks_per_seq,
    uint32_t num_blocks, int table_cap, int stages, float scale, int* status, AttRope rope) {
    constexpr int NH = D / 64;                       // 128-byte rows per token
    constexpr int STATE = D + 2;
    constexpr int KSTEPS = D / 16;
    constexpr int NTILES = D / 8;
    extern __shared__ __align__(128) unsigned char att_smem[];
    const int nwarps = int(blockDim.x >> 5) - 1;     // consumer warps; the last warp is the producer
    const uint32_t chunk = uint32_t(block_size) * D * 2;                   // bytes of one block's K (or V) for one kv head
    const uint32_t half_bytes = uint32_t(block_size) * 128;                // one 64-dim half of it: [token][128 bytes], swizzled
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(att_smem) + 1023) & ~uintptr_t(1023));
    float* warp_part = reinterpret_cast<float*>(ring);                     // aliases the ring once it is drained
    const size_t ring_bytes = max(size_t(stages) * 2 * chunk, size_t(nwarps) * G * STATE * sizeof(float));
    float* cl_part = reinterpret_cast<float*>(ring + ((ring_bytes + 127) & ~size_t(127)));        // [nsplit<=8][G][STATE]
    uint32_t* blocks = reinterpret_cast<uint32_t*>(cl_part + ATT_SPLITS * G * STATE);
    uint64_t* bars = reinterpret_cast<uint64_t*>(blocks + ((table_cap + 1) & ~1));                // full[stages], empty[stages]

    pdl_trigger();
    uint32_t nsplit;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nsplit));
    const int split = int(att_cluster_rank());
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    long long kv_len_raw = seq_used_k[b];
    const long long kv_cap = (long long)max_blocks_per_seq * block_size;
    if (kv_len_raw > kv_cap) {
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_BLOCK);
        kv_len_raw = kv_cap;
    }
    const int kv_len = int(kv_len_raw);
    const int total_blk = (kv_len + block_size - 1) / block_size;
    const int per = (total_blk + int(nsplit) - 1) / int(nsplit);
    const int first_blk = min(split * per, total_blk);
    int nblk = min(per, total_blk - first_blk);
    if (nblk > table_cap) {
        if (threadIdx.x == 0) atomicCAS(status, 0, DEV_BAD_BLOCK);
        nblk = 0;
    }
    for (int i = threadIdx.x; i < nblk; i += int(blockDim.x)) {
        uint32_t pb = block_table[size_t(b) * max_blocks_per_seq + first_blk + i];
        if (pb >= num_blocks) {                                            // never copy from outside the cache
            atomicCAS(status, 0, DEV_BAD_BLOCK);
            pb = 0;
        }
        blocks[i] = pb;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[stages + s]), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    // What the previous kernels of the stream produce for this one is q and the cache slot of the newest token
    // (position kv_len - 1, in the sequence's last block).  Every other cache block was written in earlier steps,
    // so the producer starts streaming them at once and only the last block, and the consumers' q, wait.
    const int newest_blk = total_blk - 1;

    if (warp == nwarps) {
        // ---------------- producer: lane s owns ring stage s and issues, in order, every block that passes
        // through it (a single thread's TMA issue rate would otherwise bound short sequences).  Consumer warp
        // w owns stages [w*spw, (w+1)*spw) and takes blocks w, w+nwarps, ...; its j-th block sits in stage
        // w*spw + j%spw.  Each side waits on one barrier strictly in phase order, so a parity wait is never
        // more than one phase ahead of its barrier.
        const int spw = stages / nwarps;
        if (lane < stages) {
            const int w = lane / spw, r = lane - w * spw;
            const uint32_t full = smem_u32(&bars[lane]);
            const uint32_t dst = smem_u32(ring + size_t(lane) * 2 * chunk);
            bool waited = false;
            for (int n = 0;; ++n) {
                const int i = w + nwarps * (r + spw * n);
                if (i >= nblk) break;
                if (!rope.enabled && !waited && first_blk + i >= newest_blk) {
                    pdl_wait();                    // (with the append folded in, no preceding kernel writes the cache)
                    waited = true;
                }
                if (n >= 1 && !mbar_wait(smem_u32(&bars[stages + lane]), uint32_t((n - 1) & 1), status, ATT_ERR_EMPTY)) break;
                const int token0 = int((blocks[i] * uint32_t(num_kv_heads) + uint32_t(kvh)) * uint32_t(block_size));
                mbar_arrive_expect_tx(full, 2 * chunk);
#pragma unroll
                for (int h = 0; h < NH; ++h) {                              // [half][token][128 bytes]: ldmatrix rows 8 tokens apart never share a bank
                    tma_load_3d(dst + h * half_bytes, &k_map, 0, h, token0, full);
                    tma_load_3d(dst + chunk + h * half_bytes, &v_map, 0, h, token0, full);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------- consumers: warp w owns blocks w, w+8, ...
        pdl_wait();
        const int row = lane >> 2, quad = lane & 3;
        uint32_t qa0[KSTEPS], qa2[KSTEPS];             // A fragments of Q: row = query head (zero beyond G), 16 dims per step
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            qa0[kk] = qa2[kk] = 0u;
            if (row < G) {
                const uint16_t* qp = q + b * ld_q + (size_t(kvh) * G + row) * D + kk * 16 + quad * 2;
                qa0[kk] = *reinterpret_cast<const uint32_t*>(qp);
                qa2[kk] = *reinterpret_cast<const uint32_t*>(qp + 8);
            }
        }
        if (rope.enabled) {
            const uint32_t pos = rope.positions[b];
            if (pos >= rope.max_pos) {
                if (lane == 0) atomicCAS(status, 0, DEV_BAD_POSITION);
            } else if (row < G) {
                const float* cs = rope.cos_table + size_t(pos) * D;
                const float* sn = rope.sin_table + size_t(pos) * D;
#pragma unroll
                for (int kk = 0; kk < KSTEPS / 2; ++kk) {
                    const int d = kk * 16 + quad * 2;                      // < D/2; partner dim d + D/2 sits KSTEPS/2 steps on
                    const uint32_t a0 = qa0[kk], b0 = qa0[kk + KSTEPS / 2], a2 = qa2[kk], b2 = qa2[kk + KSTEPS / 2];
                    qa0[kk] = att_rope_pair(a0, b0, cs + d, sn + d, true);
                    qa0[kk + KSTEPS / 2] = att_rope_pair(a0, b0, cs + d, sn + d, false);
                    qa2[kk] = att_rope_pair(a2, b2, cs + d + 8, sn + d + 8, true);
                    qa2[kk + KSTEPS / 2] = att_rope_pair(a2, b2, cs + d + 8, sn + d + 8, false);
                }
            }
        }
        const float sl2 = scale * 1.4426950408889634f;                     // scores live in the log2 domain
        float m2 = -INFINITY, lsum = 0.0f;                                 // this lane's row; lsum is the lane's share of the row sum
        float o[NTILES][2];
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) o[nt][0] = o[nt][1] = 0.0f;
        float z[4][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}};   // rows 8..15: always zero, rotated to keep the MMAs independent
        // ldmatrix lane roles: lane supplies the row address of matrix lane/8, row lane%8
        const int lm = lane >> 3, lr = lane & 7;
        bool alive = true;
        const int spw = stages / nwarps;
        for (int i = warp, j = 0; i < nblk && alive; i += nwarps, ++j) {
            const int s = warp * spw + j % spw;
            alive = mbar_wait(smem_u32(&bars[s]), uint32_t((j / spw) & 1), status, ATT_ERR_FULL);
            if (!alive) break;
            const uint32_t kst = smem_u32(ring + size_t(s) * 2 * chunk);
            const uint32_t vst = kst + chunk;
            const int t0 = (first_blk + i) * block_size;
            if (rope.enabled && first_blk + i == newest_blk) {
                // the newest token: rotate k_new, write it and v_new to the cache slot and into this tile
                const int slot = kv_len - 1 - t0;
                const uint32_t pos = rope.positions[b];
                const size_t cache_off = ((size_t(blocks[i]) * num_kv_heads + kvh) * block_size + slot) * D;
                unsigned char* ktile = ring + size_t(s) * 2 * chunk;
                // a block id outside the cache was replaced by 0 for the loads (and reported): never append there
                const bool slot_ok = pos < rope.max_pos && block_table[size_t(b) * max_blocks_per_seq + newest_blk] < num_blocks;
                if (slot_ok && lane < D / 16) {
                    const int d = lane * 8;                                // dims d..d+7 pair with d + D/2 ..
                    const uint16_t* kp = rope.k_new + b * rope.ld_k + size_t(kvh) * D;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(kp + d), x1 = *reinterpret_cast<const uint4*>(kp + d + D / 2);
                    const float* cs = rope.cos_table + size_t(pos) * D + d;
                    const float* sn = rope.sin_table + size_t(pos) * D + d;
                    const uint32_t xw0[4] = {x0.x, x0.y, x0.z, x0.w}, xw1[4] = {x1.x, x1.y, x1.z, x1.w};
                    uint32_t r0[4], r1[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        r0[j] = att_rope_pair(xw0[j], xw1[j], cs + 2 * j, sn + 2 * j, true);
                        r1[j] = att_rope_pair(xw0[j], xw1[j], cs + 2 * j, sn + 2 * j, false);
                    }
                    const uint4 o0 = make_uint4(r0[0], r0[1], r0[2], r0[3]), o1 = make_uint4(r1[0], r1[1], r1[2], r1[3]);
                    *reinterpret_cast<uint4*>(rope.cache_k + cache_off + d) = o0;
                    *reinterpret_cast<uint4*>(rope.cache_k + cache_off + d + D / 2) = o1;
                    const int d1 = d + D / 2;
                    *reinterpret_cast<uint4*>(ktile + (d >> 6) * half_bytes + slot * 128 + ((((d & 63) >> 3) ^ (slot & 7)) << 4)) = o0;
                    *reinterpret_cast<uint4*>(ktile + (d1 >> 6) * half_bytes + slot * 128 + ((((d1 & 63) >> 3) ^ (slot & 7)) << 4)) = o1;
                }
                if (slot_ok && lane >= 16 && lane < 16 + D / 8) {
                    const int d = (lane - 16) * 8;
                    const uint4 vv = *reinterpret_cast<const uint4*>(rope.v_new + b * rope.ld_v + size_t(kvh) * D + d);
                    *reinterpret_cast<uint4*>(rope.cache_v + cache_off + d) = vv;
                    *reinterpret_cast<uint4*>(ktile + chunk + (d >> 6) * half_bytes + slot * 128 + ((((d & 63) >> 3) ^ (slot & 7)) << 4)) = vv;
                }
                __syncwarp();                                              // the patched tile is read by this warp's ldmatrix
            }
            for (int sub = 0; sub < block_size; sub += 16) {
                if (t0 + sub >= kv_len) break;
                // S[16 x 16 tokens] = Q K^T
                float sc[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    // matrices: (tokens 0-7, dims +0..7), (tokens 0-7, dims +8..15), (tokens 8-15, +0..7), (tokens 8-15, +8..15)
                    const int token = sub + (lm >> 1) * 8 + lr;
                    const int dchunk = kk * 2 + (lm & 1);                  // 16-byte piece of the token's D*2-byte row
                    uint32_t kb[4];
                    ldsm_x4(kst + (dchunk >> 3) * half_bytes + token * 128 + (((dchunk & 7) ^ (token & 7)) << 4), kb);
                    mma_bf16_16816(sc[0][0], sc[0][1], z[0][0], z[0][1], qa0[kk], qa2[kk], kb[0], kb[1]);
                    mma_bf16_16816(sc[1][0], sc[1][1], z[1][0], z[1][1], qa0[kk], qa2[kk], kb[2], kb[3]);
                }
                // online softmax on the row this lane holds (tokens j*8 + quad*2 + {0,1})
                float rmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const bool valid = t0 + sub + j * 8 + quad * 2 + e < kv_len;
                        sc[j][e] = valid ? sc[j][e] * sl2 : -INFINITY;
                        rmax = fmaxf(rmax, sc[j][e]);
                    }
                }
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
                const float mn = fmaxf(m2, rmax);                          // finite: token t0+sub is valid
                const float corr = fast_exp2(m2 - mn);                     // 0 on the first tile (m2 = -inf)
                m2 = mn;
                float p[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    p[j][0] = fast_exp2(sc[j][0] - mn);
                    p[j][1] = fast_exp2(sc[j][1] - mn);
                }
                lsum = lsum * corr + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int nt = 0; nt < NTILES; ++nt) {
                        o[nt][0] *= corr;
                        o[nt][1] *= corr;
                    }
                }
                // P as the A operand of the second product: k = tokens; bf16 head + bf16 remainder
                const uint32_t ph0 = pack_bf16x2(p[0][0], p[0][1]), ph2 = pack_bf16x2(p[1][0], p[1][1]);
                const uint32_t pl0 = pack_bf16x2(p[0][0] - bf16_bits_to_f32(ph0 & 0xFFFFu), p[0][1] - __uint_as_float(ph0 & 0xFFFF0000u));
                const uint32_t pl2 = pack_bf16x2(p[1][0] - bf16_bits_to_f32(ph2 & 0xFFFFu), p[1][1] - __uint_as_float(ph2 & 0xFFFF0000u));
#pragma unroll
                for (int nt = 0; nt < NTILES; nt += 2) {
                    // matrices: (tokens 0-7, dims nt*8..), (tokens 8-15, dims nt*8..), (tokens 0-7, dims (nt+1)*8..), (tokens 8-15, ...)
                    const int token = sub + (lm & 1) * 8 + lr;
                    const int dchunk = nt + (lm >> 1);
                    uint32_t vb[4];
                    ldsm_x4_trans(vst + (dchunk >> 3) * half_bytes + token * 128 + (((dchunk & 7) ^ (token & 7)) << 4), vb);
                    mma_bf16_16816(o[nt][0], o[nt][1], z[0][0], z[0][1], ph0, ph2, vb[0], vb[1]);
                    mma_bf16_16816(o[nt + 1][0], o[nt + 1][1], z[1][0], z[1][1], ph0, ph2, vb[2], vb[3]);
                    mma_bf16_16816(o[nt][0], o[nt][1], z[2][0], z[2][1], pl0, pl2, vb[0], vb[1]);
                    mma_bf16_16816(o[nt + 1][0], o[nt + 1][1], z[3][0], z[3][1], pl0, pl2, vb[2], vb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[stages + s]));
        }
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
        // every warp is past its last ring read before warp_part (which aliases the ring) is written;
        // the blocks another warp still waits for are that warp's own
        asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32) : "memory");
        if (row < G) {
            float* st = warp_part + (warp * G + row) * STATE;
#pragma unroll
            for (int nt = 0; nt < NTILES; ++nt) {
                st[nt * 8 + quad * 2] = o[nt][0];
                st[nt * 8 + quad * 2 + 1] = o[nt][1];
            }
            if (quad == 0) {
                st[D] = m2 * 0.6931471805599453f;                          // back to the natural-log domain of the merge
                st[D + 1] = lsum;
            }
        }
        att_cta_merge<D>(G, nwarps, warp_part, cl_part, split, int(nsplit), kvh * G, b, out, ld_o);
    }
    if (nsplit > 1) {
        att_cluster_sync();
        if (split == 0) att_cluster_finish<D>(G, cl_part, int(nsplit), kvh * G, b, out, ld_o, int(blockDim.x));
    }
}

// Bytes of dynamic shared memory one CTA may take so that two CTAs fit on an SM.
constexpr size_t ATT_SMEM_BUDGET = 110 * 1024;
constexpr size_t ATT_SMEM_BUDGET_ALONE = 200 * 1024;
constexpr int ATT_MAX_STAGES = 24;

template <int D, int G>
cudaError_t attention_launch(const uint16_t* q, long long ld_q, const uint16_t* cache_k, const uint16_t* cache_v,
                             const uint32_t* block_table, const uint32_t* seq_used_k, uint16_t* out, long long ld_o, int batch,
                             int num_kv_heads, int block_size, int max_blocks_per_seq, uint32_t num_blocks, float scale,
                             int sm_count, int* status, cudaStream_t stream, const AttRope& rope) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cfg.stream = stream;

    // streaming variant: blocks of a multiple of 16 tokens (one TMA box, 16-token MMA tiles), two ring stages in the budget
    const size_t chunk = size_t(block_size) * D * 2;
    const size_t part = size_t(ATT_SPLITS) * G * (D + 2) * sizeof(float);
    const size_t warp_part = size_t(ATT_WARPS) * G * (D + 2) * sizeof(float);
    int nsplit = ATT_SPLITS;                         // the most splits that still run as a single wave of two CTAs per SM
    while (nsplit > 1 && (long long)batch * num_kv_heads * nsplit > 2LL * sm_count) nsplit /= 2;
    const int table_cap = max_blocks_per_seq / nsplit + 2;
    const size_t fixed = part + size_t((table_cap + 1) & ~1) * 4 + 2 * ATT_MAX_STAGES * sizeof(uint64_t) + 1024 + 128;
    // alone on its SM: 8 consumer warps and a deep ring; otherwise 4 consumer warps and about half an SM's shared
    // memory.  The big CTA (48 K registers, ~200 KB) shares its SM with no CTA of the kernels before and after it in
    // the stream, so it pays only while the grid leaves most SMs to them: up to half the SMs.  (Llama-3.2-3B decode
    // step, measured inside the step: batch 1, 64 CTAs — 1.074 ms with the big CTA, 1.116 with the small one; batch 2,
    // 128 CTAs — 1.341 ms with the big one, 1.193 with the small one.)  Every warp owns stages / warps ring stages
    // and wants at least two of them, so that its next block loads while it works on the current one.
    const bool alone = 2LL * batch * num_kv_heads * nsplit <= sm_count;
    const size_t budget = alone ? ATT_SMEM_BUDGET_ALONE : ATT_SMEM_BUDGET;
    int nwarps = alone ? 8 : 4, spw = 0;
    for (; nwarps >= 2; nwarps /= 2) {
        spw = budget > fixed ? int(std::min<size_t>(3, (budget - fixed) / (2 * chunk * nwarps))) : 0;
        if (spw >= 2) break;
    }
    if (spw < 2) {                                   // large blocks: settle for one stage per warp if that fits
        nwarps = 2;
        spw = budget > fixed ? int(std::min<size_t>(3, (budget - fixed) / (2 * chunk * nwarps))) : 0;
    }
    const unsigned long long total_tokens = (unsigned long long)num_blocks * num_kv_heads * block_size;
    tc_encode_tiled_fn enc = tc_tensor_map_encoder();
    if (enc && block_size % 16 == 0 && block_size <= 256 && total_tokens < (1ull << 31) && spw >= 1) {
        const int stages = spw * nwarps;
        const size_t ring = std::max(size_t(stages) * 2 * chunk, size_t(nwarps) * G * (D + 2) * sizeof(float));
        const size_t smem = ((ring + 127) & ~size_t(127)) + fixed;
        CUtensorMap maps[2];
        const cuuint64_t dims[3] = {64, cuuint64_t(D / 64), cuuint64_t(total_tokens)};
        const cuuint64_t strides[2] = {128, cuuint64_t(D) * 2};
        const cuuint32_t box[3] = {64, 1, cuuint32_t(block_size)};
        const cuuint32_t estr[3] = {1, 1, 1};
        const void* bases[2] = {cache_k, cache_v};
        for (int i = 0; i < 2; ++i) {
            const CUresult r = enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(bases[i]), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        }
        auto kernel = attention_decode_tc_kernel<D>;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        cfg.gridDim = dim3(nsplit, num_kv_heads, batch);
        cfg.blockDim = dim3((nwarps + 1) * 32);
        cfg.dynamicSmemBytes = smem;
        attr[0].val.clusterDim.x = nsplit;
        return cudaLaunchKernelEx(&cfg, kernel, maps[0], maps[1], q, ld_q, block_table, seq_used_k, out, ld_o, G, num_kv_heads,
                                  block_size, max_blocks_per_seq, num_blocks, table_cap, stages, scale, status, rope);
    }
    if (rope.enabled) return cudaErrorNotSupported;  // the rotation and the append are folded into the streaming variant only
    // small or odd blocks: per-token loads
    const int cap1 = max_blocks_per_seq / ATT_SPLITS + 3;
    const size_t smem = warp_part + part + size_t(cap1) * sizeof(uint32_t);
    auto kernel = attention_decode_kernel<D, G>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(ATT_SPLITS, num_kv_heads, batch);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = smem;
    attr[0].val.clusterDim.x = ATT_SPLITS;
    return cudaLaunchKernelEx(&cfg, kernel, q, ld_q, cache_k, cache_v, block_table, seq_used_k, out, ld_o, num_kv_heads,
                              block_size, max_blocks_per_seq, num_blocks, cap1, scale, status);
}

template <int D>
cudaError_t attention_dispatch_g(int G, const uint16_t* q, long long ld_q, const uint16_t* ck, const uint16_t* cv,
                                 const uint32_t* bt, const uint32_t* used, uint16_t* out, long long ld_o, int batch, int hkv,
                                 int bs, int mb, uint32_t nb, float scale, int sms, int* status, cudaStream_t st,
                                 const AttRope& rope) {
    switch (G) {
#define ATT_CASE(GG) case GG: return attention_launch<D, GG>(q, ld_q, ck, cv, bt, used, out, ld_o, batch, hkv, bs, mb, nb, scale, sms, status, st, rope)
        ATT_CASE(1); ATT_CASE(2); ATT_CASE(3); ATT_CASE(4); ATT_CASE(5); ATT_CASE(6); ATT_CASE(7); ATT_CASE(8);
#undef ATT_CASE
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

// =============================================================================== C ABI
#define DEC_REQUIRE(cond, code, ...) do { if (!(cond)) return scr_fail(ctx, code, __VA_ARGS__); } while (0)

extern "C" int32_t scr_embed_bf16(scr_ctx* ctx, const uint32_t* ids, int32_t n_ids, const uint16_t* table, int32_t vocab,
                                  int32_t hidden, uint16_t* out, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    DEC_REQUIRE(ids && table && out, SCR_E_ARG, "embed: null pointer");
    DEC_REQUIRE(n_ids >= 0 && vocab > 0 && hidden > 0 && hidden % 8 == 0, SCR_E_SHAPE, "embed: hidden=%d must be a positive multiple of 8", hidden);
    DEC_REQUIRE(scr_aligned16(table) && scr_aligned16(out), SCR_E_ALIGN, "embed: table/out not 16-byte aligned");
    if (n_ids == 0) return SCR_OK;
    cudaError_t e = launch_pdl(embed_kernel, dim3(n_ids), dim3(128), 0, (cudaStream_t)stream, ids,
                               reinterpret_cast<const uint4*>(table), uint32_t(vocab), hidden / 8, reinterpret_cast<uint4*>(out),
                               ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "embed: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "embed");
}

static int32_t norm_launch(scr_ctx* ctx, bool add, uint16_t* residual, const uint16_t* delta, const uint16_t* weight,
                           uint16_t* out, int32_t rows, int32_t hidden, float eps, void* stream) {
    DEC_REQUIRE(residual && weight && out && (!add || delta), SCR_E_ARG, "rmsnorm: null pointer");
    DEC_REQUIRE(rows >= 0 && hidden > 0 && hidden % 8 == 0, SCR_E_SHAPE, "rmsnorm: hidden=%d must be a positive multiple of 8", hidden);
    DEC_REQUIRE(scr_aligned16(residual) && scr_aligned16(weight) && scr_aligned16(out) && (!add || scr_aligned16(delta)),
                SCR_E_ALIGN, "rmsnorm: pointer not 16-byte aligned");
    const size_t smem = size_t(hidden) * sizeof(float);
    DEC_REQUIRE(smem <= 200 * 1024, SCR_E_UNSUPPORTED, "rmsnorm: hidden=%d exceeds the shared-memory row buffer", hidden);
    if (rows == 0) return SCR_OK;
    cudaError_t e = cudaSuccess;
    if (add) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e == cudaSuccess)
            e = launch_pdl(rmsnorm_kernel<true>, dim3(rows), dim3(NORM_THREADS), smem, (cudaStream_t)stream, residual, delta, weight,
                           out, hidden, eps);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e == cudaSuccess)
            e = launch_pdl(rmsnorm_kernel<false>, dim3(rows), dim3(NORM_THREADS), smem, (cudaStream_t)stream, residual,
                           (const uint16_t*)nullptr, weight, out, hidden, eps);
    }
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "rmsnorm: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "rmsnorm");
}

extern "C" int32_t scr_rmsnorm_bf16(scr_ctx* ctx, const uint16_t* x, const uint16_t* weight, uint16_t* out, int32_t rows,
                                    int32_t hidden, float eps, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    return norm_launch(ctx, false, const_cast<uint16_t*>(x), nullptr, weight, out, rows, hidden, eps, stream);
}

extern "C" int32_t scr_fused_add_rmsnorm_bf16(scr_ctx* ctx, uint16_t* residual, const uint16_t* delta, const uint16_t* weight,
                                              uint16_t* out, int32_t rows, int32_t hidden, float eps, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    return norm_launch(ctx, true, residual, delta, weight, out, rows, hidden, eps, stream);
}

static int32_t silu_mul_launch(scr_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t ld_in, uint16_t* out, int32_t rows,
                               int32_t inter, int vstride, void* stream);

extern "C" int32_t scr_silu_mul_bf16(scr_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t ld_in, uint16_t* out,
                                     int32_t rows, int32_t inter, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    return silu_mul_launch(ctx, gate, up, ld_in, out, rows, inter, 8, stream);
}

extern "C" int32_t scr_silu_mul_pairs8_bf16(scr_ctx* ctx, const uint16_t* gate_up, int64_t ld_in, uint16_t* out, int32_t rows,
                                            int32_t inter, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!gate_up) return scr_fail(ctx, SCR_E_ARG, "silu_mul: null pointer");
    if (ld_in < 2 * (int64_t)inter) return scr_fail(ctx, SCR_E_SHAPE, "silu_mul: ld_in=%lld is shorter than 2*inter", (long long)ld_in);
    return silu_mul_launch(ctx, gate_up, gate_up + 8, ld_in, out, rows, inter, 16, stream);
}

static int32_t silu_mul_launch(scr_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t ld_in, uint16_t* out, int32_t rows,
                               int32_t inter, int vstride, void* stream) {
    DEC_REQUIRE(gate && up && out, SCR_E_ARG, "silu_mul: null pointer");
    DEC_REQUIRE(rows >= 0 && inter > 0 && inter % 8 == 0 && ld_in >= inter && ld_in % 8 == 0, SCR_E_SHAPE,
                "silu_mul: inter=%d and ld_in=%lld must be multiples of 8 with ld_in >= inter", inter, (long long)ld_in);
    DEC_REQUIRE(scr_aligned16(gate) && scr_aligned16(up) && scr_aligned16(out), SCR_E_ALIGN, "silu_mul: pointer not 16-byte aligned");
    if (rows == 0) return SCR_OK;
    const long long total_v = (long long)rows * (inter / 8);
    const int threads = 256;
    const int blocks = int(std::min<long long>((total_v + threads - 1) / threads, (long long)ctx->sm_count * 8));
    cudaError_t e = launch_pdl(silu_mul_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, gate, up, (long long)ld_in,
                               out, inter / 8, total_v, vstride);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "silu_mul: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "silu_mul");
}

extern "C" int32_t scr_rope_append_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q, const uint16_t* k, int64_t ld_k,
                                        const uint16_t* v, int64_t ld_v, const uint32_t* positions, const uint32_t* slot_mapping,
                                        const float* cos_table, const float* sin_table, int32_t max_pos, uint16_t* q_out,
                                        int64_t ld_qo, uint16_t* cache_k, uint16_t* cache_v, int32_t num_blocks,
                                        int32_t num_tokens, int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim,
                                        int32_t block_size, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    DEC_REQUIRE(q && k && v && positions && slot_mapping && cos_table && sin_table && q_out && cache_k && cache_v, SCR_E_ARG,
                "rope_append: null pointer");
    DEC_REQUIRE(num_tokens >= 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && block_size > 0 &&
                    num_blocks > 0 && max_pos > 0,
                SCR_E_SHAPE, "rope_append: bad head / block geometry");
    DEC_REQUIRE(ld_q >= (int64_t)num_q_heads * head_dim && ld_qo >= (int64_t)num_q_heads * head_dim &&
                    ld_k >= (int64_t)num_kv_heads * head_dim && ld_v >= (int64_t)num_kv_heads * head_dim,
                SCR_E_SHAPE, "rope_append: a row stride is shorter than its row");
    if (num_tokens == 0) return SCR_OK;
    const int threads = std::min(256, std::max(32, ((head_dim / 2 + 31) / 32) * 32));
    cudaError_t e = launch_pdl(rope_append_kernel, dim3(num_q_heads + num_kv_heads, num_tokens), dim3(threads), 0,
                               (cudaStream_t)stream, q, (long long)ld_q, k, (long long)ld_k, v, (long long)ld_v, positions,
                               slot_mapping, cos_table, sin_table, uint32_t(max_pos), q_out, (long long)ld_qo, cache_k, cache_v,
                               uint32_t(num_blocks), num_q_heads, num_kv_heads, head_dim, block_size, ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "rope_append: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "rope_append");
}

extern "C" int32_t scr_attention_via_cache_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q, const uint16_t* cache_k,
                                                const uint16_t* cache_v, int32_t num_blocks, const uint32_t* block_table,
                                                const uint32_t* seq_used_k, uint16_t* out, int64_t ld_o, int32_t batch,
                                                int32_t num_q_heads, int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                                                int32_t max_blocks_per_seq, float attn_scale, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    DEC_REQUIRE(q && cache_k && cache_v && block_table && seq_used_k && out, SCR_E_ARG, "attention: null pointer");
    DEC_REQUIRE(batch >= 0 && num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0 && block_size > 0 &&
                    max_blocks_per_seq > 0 && num_blocks > 0,
                SCR_E_SHAPE, "attention: bad head / block geometry");
    const int G = num_q_heads / num_kv_heads;
    DEC_REQUIRE(head_dim == 64 || head_dim == 128, SCR_E_UNSUPPORTED, "attention: head_dim=%d (64 and 128 are built)", head_dim);
    DEC_REQUIRE(G <= 8, SCR_E_UNSUPPORTED, "attention: %d query heads per kv head (up to 8 are built)", G);
    DEC_REQUIRE(batch <= 65535 && num_kv_heads <= 65535, SCR_E_SHAPE, "attention: batch / kv heads exceed the grid limits");
    DEC_REQUIRE(ld_q >= (int64_t)num_q_heads * head_dim && ld_o >= (int64_t)num_q_heads * head_dim && ld_q % 8 == 0, SCR_E_SHAPE,
                "attention: a row stride is shorter than its row or not a multiple of 8");
    DEC_REQUIRE(scr_aligned16(q) && scr_aligned16(cache_k) && scr_aligned16(cache_v), SCR_E_ALIGN,
                "attention: q / cache not 16-byte aligned");
    DEC_REQUIRE(max_blocks_per_seq <= (1 << 20), SCR_E_UNSUPPORTED, "attention: block table wider than 2^20 blocks");
    if (batch == 0) return SCR_OK;
    AttRope rope = {};
    cudaError_t e;
    if (head_dim == 128)
        e = attention_dispatch_g<128>(G, q, ld_q, cache_k, cache_v, block_table, seq_used_k, out, ld_o, batch, num_kv_heads,
                                      block_size, max_blocks_per_seq, uint32_t(num_blocks), attn_scale, ctx->sm_count, ctx->dev_status,
                                      (cudaStream_t)stream, rope);
    else
        e = attention_dispatch_g<64>(G, q, ld_q, cache_k, cache_v, block_table, seq_used_k, out, ld_o, batch, num_kv_heads,
                                     block_size, max_blocks_per_seq, uint32_t(num_blocks), attn_scale, ctx->sm_count, ctx->dev_status,
                                     (cudaStream_t)stream, rope);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "attention: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "attention_via_cache");
}

extern "C" int32_t scr_rope_attention_via_cache_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q, const uint16_t* k, int64_t ld_k,
                                                     const uint16_t* v, int64_t ld_v, const uint32_t* positions,
                                                     const float* cos_table, const float* sin_table, int32_t max_pos,
                                                     uint16_t* cache_k, uint16_t* cache_v, int32_t num_blocks,
                                                     const uint32_t* block_table, const uint32_t* seq_used_k, uint16_t* out,
                                                     int64_t ld_o, int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                                     int32_t head_dim, int32_t block_size, int32_t max_blocks_per_seq,
                                                     float attn_scale, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    DEC_REQUIRE(q && k && v && positions && cos_table && sin_table && cache_k && cache_v && block_table && seq_used_k && out, SCR_E_ARG,
                "rope_attention: null pointer");
    DEC_REQUIRE(batch >= 0 && num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0 && block_size > 0 &&
                    max_blocks_per_seq > 0 && num_blocks > 0 && max_pos > 0,
                SCR_E_SHAPE, "rope_attention: bad head / block geometry");
    const int G = num_q_heads / num_kv_heads;
    DEC_REQUIRE(head_dim == 64 || head_dim == 128, SCR_E_UNSUPPORTED, "rope_attention: head_dim=%d (64 and 128 are built)", head_dim);
    DEC_REQUIRE(G <= 8, SCR_E_UNSUPPORTED, "rope_attention: %d query heads per kv head (up to 8 are built)", G);
    DEC_REQUIRE(block_size % 16 == 0 && block_size <= 256, SCR_E_UNSUPPORTED,
                "rope_attention: block_size=%d (multiples of 16 up to 256; use rope_append + attention_via_cache otherwise)", block_size);
    DEC_REQUIRE(batch <= 65535 && num_kv_heads <= 65535, SCR_E_SHAPE, "rope_attention: batch / kv heads exceed the grid limits");
    const int64_t qd = (int64_t)num_q_heads * head_dim, kd = (int64_t)num_kv_heads * head_dim;
    DEC_REQUIRE(ld_q >= qd && ld_o >= qd && ld_k >= kd && ld_v >= kd && ld_q % 8 == 0 && ld_k % 8 == 0 && ld_v % 8 == 0, SCR_E_SHAPE,
                "rope_attention: a row stride is shorter than its row or not a multiple of 8");
    DEC_REQUIRE(scr_aligned16(q) && scr_aligned16(k) && scr_aligned16(v) && scr_aligned16(cache_k) && scr_aligned16(cache_v), SCR_E_ALIGN,
                "rope_attention: q / k / v / cache not 16-byte aligned");
    DEC_REQUIRE(max_blocks_per_seq <= (1 << 20), SCR_E_UNSUPPORTED, "rope_attention: block table wider than 2^20 blocks");
    if (batch == 0) return SCR_OK;
    AttRope rope = {};
    rope.k_new = k;
    rope.v_new = v;
    rope.positions = positions;
    rope.cos_table = cos_table;
    rope.sin_table = sin_table;
    rope.cache_k = cache_k;
    rope.cache_v = cache_v;
    rope.ld_k = ld_k;
    rope.ld_v = ld_v;
    rope.max_pos = uint32_t(max_pos);
    rope.enabled = 1;
    cudaError_t e;
    if (head_dim == 128)
        e = attention_dispatch_g<128>(G, q, ld_q, cache_k, cache_v, block_table, seq_used_k, out, ld_o, batch, num_kv_heads,
                                      block_size, max_blocks_per_seq, uint32_t(num_blocks), attn_scale, ctx->sm_count, ctx->dev_status,
                                      (cudaStream_t)stream, rope);
    else
        e = attention_dispatch_g<64>(G, q, ld_q, cache_k, cache_v, block_table, seq_used_k, out, ld_o, batch, num_kv_heads,
                                     block_size, max_blocks_per_seq, uint32_t(num_blocks), attn_scale, ctx->sm_count, ctx->dev_status,
                                     (cudaStream_t)stream, rope);
    if (e == cudaErrorNotSupported) {
        (void)cudaGetLastError();
        return scr_fail(ctx, SCR_E_UNSUPPORTED, "rope_attention: this geometry has no streaming variant (use rope_append + attention_via_cache)");
    }
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "rope_attention: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "rope_attention_via_cache");
}

extern "C" int32_t scr_argmax_bf16(scr_ctx* ctx, const uint16_t* logits, int64_t ld, int32_t rows, int32_t width, uint32_t* out,
                                   void* stream) {
    SCR_REQUIRE_CTX(ctx);
    DEC_REQUIRE(logits && out, SCR_E_ARG, "argmax: null pointer");
    DEC_REQUIRE(rows >= 0 && width > 0 && ld >= width && ld % 8 == 0, SCR_E_SHAPE,
                "argmax: width=%d, ld=%lld (ld must be a multiple of 8, at least width)", width, (long long)ld);
    DEC_REQUIRE(scr_aligned16(logits), SCR_E_ALIGN, "argmax: logits not 16-byte aligned");
    if (rows == 0) return SCR_OK;
    cudaError_t e = launch_pdl(argmax_kernel, dim3(rows), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, logits, (long long)ld,
                               width, out);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "argmax: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "argmax");
}
