// Context lifecycle, status strings and the workspace query of the C ABI.
#include "common.cuh"
#include <new>

size_t affine_workspace_bytes(int M, int N, int K);
size_t fp8_workspace_bytes(int M, int N, int K);

extern "C" const char* scr_status_string(int32_t s) {
    switch (s) {
        case SCR_OK: return "SCR_OK";
        case SCR_E_ARG: return "SCR_E_ARG";
        case SCR_E_SHAPE: return "SCR_E_SHAPE";
        case SCR_E_ALIGN: return "SCR_E_ALIGN";
        case SCR_E_DTYPE: return "SCR_E_DTYPE";
        case SCR_E_CUDA: return "SCR_E_CUDA";
        case SCR_E_WORKSPACE: return "SCR_E_WORKSPACE";
        case SCR_E_UNSUPPORTED: return "SCR_E_UNSUPPORTED";
        case SCR_E_TIMEOUT: return "SCR_E_TIMEOUT";
        case SCR_E_COMM: return "SCR_E_COMM";
        default: return "SCR_E_UNKNOWN";
    }
}

extern "C" const char* scr_last_error(const scr_ctx* ctx) { return ctx ? ctx->err : "null context"; }

extern "C" int32_t scr_cuda_init(int32_t device, scr_ctx** out) {
    if (!out) return SCR_E_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return SCR_E_CUDA;
    if (device < 0 || device >= count) return SCR_E_ARG;
    if (cudaSetDevice(device) != cudaSuccess) return SCR_E_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return SCR_E_CUDA;
    if (prop.major != 10) return SCR_E_UNSUPPORTED;   // the kernels are sm_100a only
    scr_ctx* c = new (std::nothrow) scr_ctx();
    if (!c) return SCR_E_CUDA;
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;
    if (cudaMalloc((void**)&c->dev_status, sizeof(int)) != cudaSuccess || cudaMemset(c->dev_status, 0, sizeof(int)) != cudaSuccess) {
        delete c;
        return SCR_E_CUDA;
    }
    *out = c;
    return SCR_OK;
}

extern "C" int32_t scr_cuda_destroy(scr_ctx* ctx) {
    if (!ctx) return SCR_E_ARG;
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    delete ctx;
    return SCR_OK;
}

extern "C" int64_t scr_launch_count(const scr_ctx* ctx) { return ctx ? (int64_t)ctx->launches.load() : 0; }

extern "C" int32_t scr_linear_workspace_size(int32_t kind, int32_t M, int32_t N, int32_t K, size_t* bytes) {
    if (!bytes) return SCR_E_ARG;
    if (M <= 0 || N <= 0 || K <= 0) return SCR_E_SHAPE;
    if (kind == SCR_KIND_AFFINE_B4) { *bytes = affine_workspace_bytes(M, N, K); return SCR_OK; }
    if (kind == SCR_KIND_FP8_DYNAMIC) { *bytes = fp8_workspace_bytes(M, N, K); return SCR_OK; }
    return SCR_E_ARG;
}

extern "C" int32_t scr_device_status(scr_ctx* ctx, void* stream, int32_t* code) {
    SCR_REQUIRE_CTX(ctx);
    int host = 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(&host, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "device status read: %s", cudaGetErrorString(e));
    if (code) *code = host;
    if (host != 0) {
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), st);
        if ((host >> 24) == 0x0E)
            return scr_fail(ctx, SCR_E_ARG, "a device-side argument check failed (code 0x%08x: %s out of range)", host,
                            host == 0x0E000001 ? "token id" : host == 0x0E000002 ? "cache slot" : host == 0x0E000003 ? "block id / kv length" : "position");
        return scr_fail(ctx, SCR_E_TIMEOUT, "a bounded device-side wait ran out (code %d)", host);
    }
    return SCR_OK;
}

__global__ void partial_to_bf16_kernel(const float* __restrict__ in, long long count, uint16_t* __restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const __nv_bfloat16 v = __float2bfloat16_rn(in[i]);
        out[i] = *reinterpret_cast<const uint16_t*>(&v);
    }
}

extern "C" int32_t scr_partial_to_bf16(scr_ctx* ctx, const float* in, int64_t count, uint16_t* out, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!in || !out) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (count <= 0) return SCR_OK;
    const int threads = 256;
    const int blocks = (int)std::min<long long>((count + threads - 1) / threads, (long long)ctx->sm_count * 8);
    partial_to_bf16_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(in, (long long)count, out);
    return scr_check_launch(ctx, "partial_to_bf16");
}
