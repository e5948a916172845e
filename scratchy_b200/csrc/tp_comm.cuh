// Shared pieces of the tensor-parallel exchange over NVLink peer memory: the communicator object, the peer
// pointer table a kernel receives, and the system-scope publish / poll helpers.  Used by the stand-alone
// all-reduce kernel (tp_comm.cu) and by the row-parallel matvec that pushes and sums in its own epilogue (fp8.cu).
#pragma once
#include "common.cuh"

#define TPC_MAX_WORLD 8
#define TPC_MAX_GRID 256                     // grid of the stand-alone all-reduce kernel
#define TPC_THREADS 256
#define TPC_SLICE (TPC_THREADS * 4)          // f32 elements one CTA moves per pass
#define TPC_WAIT_LIMIT (1u << 22)
#define TPC_ERR_FLAG_WAIT 0x0C000001

// Every exchanged value travels as an 8-byte packet {f32 bits, call number}: an aligned 8-byte store is
// single-copy atomic, so a receiver that reads the expected call number has the value with it — no
// system-scope fence and no separate flag on either side (a fence.sys costs microseconds; measured).
// Larger payloads (more than TPC_PACKET_MAX values summed over the ranks) go the other way: dense f32 stores into
// a second receive area, then one flag per CTA and rank with release / acquire at system scope — half the bytes
// and 16-byte stores; the two fences are then small against the transfer (TP=8, 32 tokens: 156 us per layer
// against 332 us with packets).
#define TPC_PACKET_MAX 32768
#define TPC_MAX_CTAS 256                     // flag slots per (half, rank)
// Payloads of TPC_TWO_PHASE_MIN values and more (prefill chunks) are bandwidth, not latency: pushing every rank's whole
// partial to every rank moves (W-1) * 4 bytes per element and rank.  The two-phase kernel moves (W-1)/W * (4 + 2):
// each rank receives only its 1/W slice of the others' f32 partials, sums the W copies in rank order, rounds once and
// pushes the bf16 slice to everybody (a reduce-scatter and an all-gather inside one kernel, plain peer stores).
#define TPC_TWO_PHASE_MIN 131072
#define TPC_ONE_SHOT_MAX 524288              // capacity of the one-shot areas (64 tokens x 8192)
struct TpcPeers {
    uint2* ll[TPC_MAX_WORLD];                // base of each rank's packet area   [2][W][one_elems] packets
    float* recv[TPC_MAX_WORLD];              // base of each rank's dense area    [2][W][one_elems] f32
    unsigned int* flags[TPC_MAX_WORLD];      // base of each rank's flag area     [2][W][TPC_MAX_CTAS]
    float* rs[TPC_MAX_WORLD];                // two-phase: slices received        [2][W][slice_max] f32
    uint16_t* ag[TPC_MAX_WORLD];             // two-phase: the gathered result    [2][max_elems] bf16
    unsigned int* flags2[TPC_MAX_WORLD];     // two-phase: flags                  [2 phases][2][W][TPC_MAX_CTAS]
};

struct scr_tp_comm {
    scr_ctx* ctx = nullptr;
    int world = 1, rank = 0;
    long long max_elems = 0;                 // largest count of a call
    long long one_elems = 0;                 // capacity (and stride) of the one-shot areas: min(max_elems, TPC_ONE_SHOT_MAX)
    long long slice_max = 0;                 // two-phase: ceil(max_elems / world), a multiple of 8
    size_t bytes = 0, recv_off = 0, flags_off = 0, rs_off = 0, ag_off = 0, flags2_off = 0;
    unsigned char* local = nullptr;
    unsigned char* peer[TPC_MAX_WORLD] = {nullptr};
    bool opened[TPC_MAX_WORLD] = {false};
    unsigned int* state = nullptr;           // device: [0] = call counter, [1] = CTAs finished in the running call
    unsigned int wait_limit = TPC_WAIT_LIMIT;    // polls a kernel waits for a peer's packet or flag before it gives up
    bool connected = false;
};

// What a kernel that exchanges in its own epilogue needs (passed by value).
struct TpcExchange {
    TpcPeers peers;
    int world, rank;
    long long max_elems;
    unsigned int* state;
    uint16_t* y_bf16;                        // the reduced, rounded result [M, N]
    unsigned int wait_limit;
};

static inline TpcPeers tpc_peer_table(const scr_tp_comm* comm) {
    TpcPeers peers;
    for (int p = 0; p < TPC_MAX_WORLD; ++p) {
        unsigned char* base = comm->peer[p < comm->world ? p : comm->rank];
        peers.ll[p] = reinterpret_cast<uint2*>(base);
        peers.recv[p] = reinterpret_cast<float*>(base + comm->recv_off);
        peers.flags[p] = reinterpret_cast<unsigned int*>(base + comm->flags_off);
        peers.rs[p] = reinterpret_cast<float*>(base + comm->rs_off);
        peers.ag[p] = reinterpret_cast<uint16_t*>(base + comm->ag_off);
        peers.flags2[p] = reinterpret_cast<unsigned int*>(base + comm->flags2_off);
    }
    return peers;
}

// Slot of (call e, sending rank r, element i) in a receive area: calls alternate between two halves.
__device__ __forceinline__ long long tpc_slot(unsigned int e, int world, int r, long long max_elems, long long i) {
    return ((long long)(e & 1u) * world + r) * max_elems + i;
}
// One 64-bit store and one 64-bit load per packet: a single aligned 8-byte access is single-copy atomic in the
// memory model (a vector access is modelled as separate scalar accesses and promises nothing of the kind).
__device__ __forceinline__ void tpc_ll_store(uint2* p, float v, unsigned int e) {
    const unsigned long long w = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// Bounded wait for the packet of call e: gives up (recording the code) after `limit` polls, or as soon as another
// waiter has recorded a failure, and returns 0 then — the kernel runs to its end, nothing hangs.
__device__ __forceinline__ float tpc_ll_wait(const uint2* p, unsigned int e, int* status, unsigned int limit) {
    for (unsigned int it = 0; it < limit; ++it) {
        unsigned long long w;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
        if ((unsigned int)(w >> 32) == e) return __uint_as_float((unsigned int)w);
        if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) return 0.f;
    }
    atomicCAS(status, 0, TPC_ERR_FLAG_WAIT);
    return 0.f;
}
__device__ __forceinline__ void tpc_st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int tpc_ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// The last CTA of a launch advances the call counter (every CTA has read it by then).
__device__ __forceinline__ void tpc_finish_call(unsigned int* state, unsigned int e, unsigned int ctas) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&state[1], 1u);
        if (done == ctas - 1) {
            state[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(&state[0]) = e;
        }
    }
}
