// Context, status text, options, scratch management and the fp32 peak probe.
#include <new>

#include "common.cuh"

int dlspm_cuda_fail(dlspm_ctx *ctx, cudaError_t err, const char *what)
{
    if (ctx) {
        snprintf(ctx->last_error, sizeof(ctx->last_error), "%s: %s (%s)", what,
                 cudaGetErrorString(err), cudaGetErrorName(err));
    }
    // Clear the sticky-free error state so that a later, unrelated call does not report it.
    (void)cudaGetLastError();
    return DLSPM_ERR_CUDA;
}

extern "C" const char *dlspm_strerror(int status)
{
    switch (status) {
    case DLSPM_OK: return "ok";
    case DLSPM_ERR_INVALID_ARGUMENT: return "invalid argument";
    case DLSPM_ERR_CUDA: return "CUDA runtime error";
    case DLSPM_ERR_IO: return "Error opening file!";
    case DLSPM_ERR_FORMAT: return "malformed .smtx text";
    case DLSPM_ERR_CSR: return "CSR structure failed the sanity check";
    case DLSPM_ERR_NOMEM: return "out of memory";
    case DLSPM_ERR_UNSUPPORTED: return "size beyond a documented limit";
    case DLSPM_ERR_NO_DEVICE: return "no usable CUDA device";
    case DLSPM_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
    default: return "unknown status";
    }
}

// measured crossover: the tiled kernel wins from about 45 % nonzeros
static constexpr int kDefaultTileMinDensity = 450;

extern "C" int dlspm_create(dlspm_ctx **out, int device)
{
    if (!out || device < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return DLSPM_ERR_NO_DEVICE;
    }
    if (device >= count) return DLSPM_ERR_NO_DEVICE;
    dlspm_ctx *ctx = new (std::nothrow) dlspm_ctx();
    if (!ctx) return DLSPM_ERR_NOMEM;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->tile_min_density_permille = kDefaultTileMinDensity;
    cudaDeviceProp prop;
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        (void)cudaGetLastError();
        delete ctx;
        return DLSPM_ERR_NO_DEVICE;
    }
    // The kernels are built for sm_100a only; any other device cannot run them.
    if (prop.major != 10) {
        delete ctx;
        return DLSPM_ERR_NO_DEVICE;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->global_mem = prop.totalGlobalMem;
    snprintf(ctx->name, sizeof(ctx->name), "%s", prop.name);
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        (void)cudaGetLastError();
        delete ctx;
        return DLSPM_ERR_CUDA;
    }
    *out = ctx;
    return DLSPM_OK;
}

extern "C" int dlspm_destroy(dlspm_ctx *ctx)
{
    if (!ctx) return DLSPM_OK;
    cudaSetDevice(ctx->device);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stage) cudaFree(ctx->stage);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->side_ready) {
        for (int i = 0; i < kSideStreams; i++) {
            cudaStreamDestroy(ctx->side_stream[i]);
            cudaEventDestroy(ctx->side_join[i]);
        }
        cudaEventDestroy(ctx->side_fork);
    }
    if (ctx->pipeline_ready) {
        cudaStreamDestroy(ctx->h2d_stream);
        cudaStreamDestroy(ctx->d2h_stream);
        for (int i = 0; i < kPipeSlots; i++) {
            cudaEventDestroy(ctx->ev_h2d[i]);
            cudaEventDestroy(ctx->ev_kernel[i]);
            cudaEventDestroy(ctx->ev_d2h[i]);
        }
    }
    (void)cudaGetLastError();
    delete ctx;
    return DLSPM_OK;
}

extern "C" const char *dlspm_last_error(const dlspm_ctx *ctx) { return ctx ? ctx->last_error : ""; }

extern "C" int dlspm_device_info(const dlspm_ctx *ctx, char *name, size_t name_len, int *sm_count,
                                 size_t *global_mem_bytes)
{
    if (!ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    if (name && name_len) snprintf(name, name_len, "%s", ctx->name);
    if (sm_count) *sm_count = ctx->sm_count;
    if (global_mem_bytes) *global_mem_bytes = ctx->global_mem;
    return DLSPM_OK;
}

extern "C" int dlspm_set_option(dlspm_ctx *ctx, int option, int value)
{
    if (!ctx) return DLSPM_ERR_INVALID_ARGUMENT;
    switch (option) {
    case DLSPM_OPT_STRICT_FP32: ctx->strict_fp32 = value ? 1 : 0; return DLSPM_OK;
    case DLSPM_OPT_SPMM_KERNEL:
        if (value < 0 || value > 3) return DLSPM_ERR_INVALID_ARGUMENT;
        ctx->spmm_kernel = value;
        return DLSPM_OK;
    case DLSPM_OPT_CHECK_INPUT: ctx->check_input = value ? 1 : 0; return DLSPM_OK;
    case DLSPM_OPT_TILE_MIN_DENSITY:
        if (value == -1) {  // back to the default, as if never set
            ctx->tile_min_density_permille = kDefaultTileMinDensity;
            ctx->tile_min_density_set = 0;
            return DLSPM_OK;
        }
        if (value < 0 || value > 1001) return DLSPM_ERR_INVALID_ARGUMENT;
        ctx->tile_min_density_permille = value;
        ctx->tile_min_density_set = 1;
        return DLSPM_OK;
    default: return DLSPM_ERR_INVALID_ARGUMENT;
    }
}

extern "C" int dlspm_get_option(const dlspm_ctx *ctx, int option, int *value)
{
    if (!ctx || !value) return DLSPM_ERR_INVALID_ARGUMENT;
    switch (option) {
    case DLSPM_OPT_STRICT_FP32: *value = ctx->strict_fp32; return DLSPM_OK;
    case DLSPM_OPT_SPMM_KERNEL: *value = ctx->spmm_kernel; return DLSPM_OK;
    case DLSPM_OPT_TILE_MIN_DENSITY: *value = ctx->tile_min_density_permille; return DLSPM_OK;
    case DLSPM_OPT_CHECK_INPUT: *value = ctx->check_input; return DLSPM_OK;
    default: return DLSPM_ERR_INVALID_ARGUMENT;
    }
}

static int reserve(dlspm_ctx *ctx, void **buf, size_t *have, size_t bytes)
{
    if (bytes <= *have) return DLSPM_OK;
    if (*buf) {
        // Work queued on any stream may still read the old buffer.
        DLSPM_CUDA_TRY(ctx, cudaDeviceSynchronize());
        DLSPM_CUDA_TRY(ctx, cudaFree(*buf));
        *buf = nullptr;
        *have = 0;
    }
    size_t want = bytes + bytes / 4 + 256;
    cudaError_t err = cudaMalloc(buf, want);
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "cudaMalloc(scratch)");
        *buf = nullptr;
        return DLSPM_ERR_NOMEM;
    }
    *have = want;
    return DLSPM_OK;
}

int dlspm_scratch_reserve(dlspm_ctx *ctx, size_t bytes)
{
    return reserve(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes);
}
int dlspm_stage_reserve(dlspm_ctx *ctx, size_t bytes)
{
    return reserve(ctx, &ctx->stage, &ctx->stage_bytes, bytes);
}

extern "C" void dlspm_free_host(void *p) { free(p); }

// ---- fp32 FMA peak --------------------------------------------------------------------------
// Eight independent FMA chains per thread, registers only.  The result is written only if it
// is a value it can never be, which keeps the compiler from deleting the loop.
__global__ void __launch_bounds__(256) fma_peak_kernel(float *sink, int iters, float seed)
{
    float a0 = seed + threadIdx.x, a1 = a0 + 1.f, a2 = a0 + 2.f, a3 = a0 + 3.f;
    float a4 = a0 + 4.f, a5 = a0 + 5.f, a6 = a0 + 6.f, a7 = a0 + 7.f;
    const float m = 0.999f, c = 0.001f;
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int u = 0; u < 8; u++) {
            a0 = fmaf(a0, m, c); a1 = fmaf(a1, m, c); a2 = fmaf(a2, m, c); a3 = fmaf(a3, m, c);
            a4 = fmaf(a4, m, c); a5 = fmaf(a5, m, c); a6 = fmaf(a6, m, c); a7 = fmaf(a7, m, c);
        }
    }
    float s = a0 + a1 + a2 + a3 + a4 + a5 + a6 + a7;
    if (s == -12345.678f) sink[0] = s;
}

// The same with packed multiply-adds (fma.rn.f32x2): two per instruction.
__global__ void __launch_bounds__(256) fma2_peak_kernel(float *sink, int iters, float seed)
{
    float2 a0 = make_float2(seed + threadIdx.x, seed), a1 = make_float2(a0.x + 1.f, 1.f), a2 = make_float2(a0.x + 2.f, 2.f),
           a3 = make_float2(a0.x + 3.f, 3.f);
    const float2 m = make_float2(0.999f, 0.998f), c = make_float2(0.001f, 0.002f);
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int u = 0; u < 8; u++) {
            a0 = __ffma2_rn(a0, m, c); a1 = __ffma2_rn(a1, m, c); a2 = __ffma2_rn(a2, m, c); a3 = __ffma2_rn(a3, m, c);
        }
    }
    const float s = a0.x + a0.y + a1.x + a1.y + a2.x + a2.y + a3.x + a3.y;
    if (s == -12345.678f) sink[0] = s;
}

extern "C" int dlspm_measure_fp32_peaks(dlspm_ctx *ctx, double *scalar_tflops, double *packed_tflops)
{
    if (!ctx || !scalar_tflops || !packed_tflops) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_measure_fp32_peak(ctx, scalar_tflops);
    if (rc) return rc;
    const int iters = 4096;
    const int blocks = ctx->sm_count * 8;
    cudaEvent_t e0, e1;
    DLSPM_CUDA_TRY(ctx, cudaEventCreate(&e0));
    DLSPM_CUDA_TRY(ctx, cudaEventCreate(&e1));
    float best_ms = 1e30f;
    for (int rep = 0; rep < 5; rep++) {
        cudaEventRecord(e0, ctx->stream);
        fma2_peak_kernel<<<blocks, 256, 0, ctx->stream>>>((float *)ctx->scratch, iters, 1.0f);
        cudaEventRecord(e1, ctx->stream);
        DLSPM_CUDA_TRY(ctx, cudaEventSynchronize(e1));
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best_ms) best_ms = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    // 4 chains x 2 lanes x 8 unrolled = 64 multiply-adds per thread and iteration, as in the scalar probe
    *packed_tflops = 2.0 * 64.0 * (double)iters * 256.0 * (double)blocks / (best_ms * 1e-3) * 1e-12;
    return DLSPM_OK;
}

extern "C" int dlspm_measure_fp32_peak(dlspm_ctx *ctx, double *tflops)
{
    if (!ctx || !tflops) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = dlspm_scratch_reserve(ctx, 256);
    if (rc) return rc;
    const int iters = 4096;
    const int blocks = ctx->sm_count * 8;
    cudaEvent_t e0, e1;
    DLSPM_CUDA_TRY(ctx, cudaEventCreate(&e0));
    DLSPM_CUDA_TRY(ctx, cudaEventCreate(&e1));
    float best_ms = 1e30f;
    for (int rep = 0; rep < 5; rep++) {
        cudaEventRecord(e0, ctx->stream);
        fma_peak_kernel<<<blocks, 256, 0, ctx->stream>>>((float *)ctx->scratch, iters, 1.0f);
        cudaEventRecord(e1, ctx->stream);
        DLSPM_CUDA_TRY(ctx, cudaEventSynchronize(e1));
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best_ms) best_ms = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    const double flops = 2.0 * 64.0 * (double)iters * 256.0 * (double)blocks;
    *tflops = flops / (best_ms * 1e-3) * 1e-12;
    return DLSPM_OK;
}

// ---- peer memory: buffers other GPUs (same or other process) can store into ---------------------
extern "C" int dlspm_enable_peer_access(dlspm_ctx *ctx, int peer_device)
{
    if (!ctx || peer_device < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (peer_device == ctx->device) return DLSPM_OK;
    int can = 0;
    DLSPM_CUDA_TRY(ctx, cudaDeviceCanAccessPeer(&can, ctx->device, peer_device));
    if (!can) return DLSPM_ERR_UNSUPPORTED;
    cudaError_t err = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (err == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return DLSPM_OK;
    }
    if (err != cudaSuccess) return dlspm_cuda_fail(ctx, err, "cudaDeviceEnablePeerAccess");
    return DLSPM_OK;
}

extern "C" int dlspm_peer_alloc(dlspm_ctx *ctx, size_t bytes, void **ptr, unsigned char handle[64])
{
    if (!ctx || !ptr || !handle || bytes == 0) return DLSPM_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaError_t err = cudaMalloc(ptr, bytes);
    if (err != cudaSuccess) {
        dlspm_cuda_fail(ctx, err, "cudaMalloc(peer buffer)");
        return DLSPM_ERR_NOMEM;
    }
    cudaIpcMemHandle_t h;
    err = cudaIpcGetMemHandle(&h, *ptr);
    if (err != cudaSuccess) {
        cudaFree(*ptr);
        *ptr = nullptr;
        return dlspm_cuda_fail(ctx, err, "cudaIpcGetMemHandle");
    }
    memcpy(handle, &h, 64);
    return DLSPM_OK;
}

extern "C" int dlspm_peer_open(dlspm_ctx *ctx, const unsigned char handle[64], void **ptr)
{
    if (!ctx || !ptr || !handle) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    DLSPM_CUDA_TRY(ctx, cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return DLSPM_OK;
}

extern "C" int dlspm_peer_close(dlspm_ctx *ctx, void *ptr)
{
    if (!ctx || !ptr) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    DLSPM_CUDA_TRY(ctx, cudaIpcCloseMemHandle(ptr));
    return DLSPM_OK;
}

extern "C" int dlspm_peer_free(dlspm_ctx *ctx, void *ptr)
{
    if (!ctx || !ptr) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    DLSPM_CUDA_TRY(ctx, cudaFree(ptr));
    return DLSPM_OK;
}

// ---- bounded-wait self-test --------------------------------------------------------------------
// Every wait inside a kernel of this library is a bounded poll that ends in a status, never a trap
// or an endless loop.  This entry point shows that path without any fault: one thread polls an
// mbarrier that nothing will ever complete, gives up after `polls` tries and reports it.
__global__ void bounded_wait_selftest_kernel(unsigned polls, int *timed_out)
{
    __shared__ unsigned long long bar;
    const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    unsigned done = 0;
    for (unsigned i = 0; i < polls && !done; i++) {
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr)
            : "memory");
    }
    *timed_out = done ? 0 : 1;
}

extern "C" int dlspm_selftest_bounded_wait(dlspm_ctx *ctx, unsigned polls, int *timed_out)
{
    if (!ctx || !timed_out || polls == 0 || polls > (1u << 20)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    rc = dlspm_scratch_reserve(ctx, 256);
    if (rc) return rc;
    DLSPM_CUDA_TRY(ctx, cudaMemsetAsync(ctx->scratch, 0, sizeof(int), ctx->stream));
    bounded_wait_selftest_kernel<<<1, 1, 0, ctx->stream>>>(polls, (int *)ctx->scratch);
    DLSPM_CUDA_TRY(ctx, cudaGetLastError());
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(timed_out, ctx->scratch, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return *timed_out ? DLSPM_ERR_TIMEOUT : DLSPM_OK;
}

// ---- CSR validation on the device -------------------------------------------------------------------
// The kernels trust the CSR arrays as the reference's do (a column index beyond K reads outside B).
// For arrays that never were on the host this is the reference's SanityCheck
// (SPMM/spmm-esimd-fromfile.cpp:36-61, plus row_offsets[0] == 0 and column >= 0) run on the device:
// status[0] = kind of the first violation found (0 = none), status[1] = where.
namespace {

enum { kCsrOk = 0, kCsrFirstOffset = 1, kCsrLastOffset = 2, kCsrDecreasing = 3, kCsrRowTooLong = 4, kCsrColumn = 5 };

__global__ void __launch_bounds__(256) csr_check_kernel(const int *__restrict__ row_offsets, const int *__restrict__ cols,
                                                       int M, int K, int nnz, int *status)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step = (long long)gridDim.x * blockDim.x;
    int kind = kCsrOk, where = 0;
    if (tid == 0) {
        if (row_offsets[0] != 0) { kind = kCsrFirstOffset; where = 0; }
        else if (row_offsets[M] != nnz) { kind = kCsrLastOffset; where = M; }
    }
    for (long long i = tid; i < M && kind == kCsrOk; i += step) {
        const int a = row_offsets[i], b = row_offsets[i + 1];
        if (b < a) { kind = kCsrDecreasing; where = (int)i; }
        else if (b - a > K) { kind = kCsrRowTooLong; where = (int)i; }
    }
    // columns are read only inside [0, nnz), whatever the offsets say
    for (long long p = tid; p < nnz && kind == kCsrOk; p += step) {
        const int c = cols[p];
        if (c < 0 || c >= K) { kind = kCsrColumn; where = (int)p; }
    }
    if (kind != kCsrOk && atomicCAS(&status[0], 0, kind) == 0) status[1] = where;
}

}  // namespace

extern "C" int dlspm_sanity_check_csr(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets,
                                      const int *column_indices, char *why, size_t why_len, void *stream)
{
    if (!ctx || M < 0 || K < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    if (why && why_len) why[0] = 0;
    if ((long long)nnz > (long long)M * (long long)K) {
        if (why && why_len) snprintf(why, why_len, "nnz is larger than matrix.");
        return DLSPM_ERR_CSR;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int *status = nullptr;
    DLSPM_CUDA_TRY(ctx, cudaMalloc(&status, 2 * sizeof(int)));
    int host[2] = {0, 0};
    cudaError_t err = cudaMemsetAsync(status, 0, 2 * sizeof(int), st);
    if (err == cudaSuccess) {
        const long long work = (long long)M > (long long)nnz ? M : nnz;
        const int blocks = (int)((work + 255) / 256 < 1 ? 1 : ((work + 255) / 256 > (long long)ctx->sm_count * 16 ? (long long)ctx->sm_count * 16 : (work + 255) / 256));
        csr_check_kernel<<<blocks, 256, 0, st>>>(row_offsets, column_indices, M, K, nnz, status);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaMemcpyAsync(host, status, sizeof(host), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    cudaFree(status);
    if (err != cudaSuccess) return dlspm_cuda_fail(ctx, err, "device CSR check");
    if (host[0] == kCsrOk) return DLSPM_OK;
    if (why && why_len) {
        // the reference's exception texts where it has one
        // the host check's texts (the reference's exception texts where it has one), plus the place
        switch (host[0]) {
        case kCsrFirstOffset: snprintf(why, why_len, "a_row_offsets[0] != 0"); break;
        case kCsrLastOffset: snprintf(why, why_len, "a_row_offsets[MSZ] != nnz."); break;
        case kCsrDecreasing: snprintf(why, why_len, "a_row_offsets[i+1] < a_row_offsets[i] (i = %d)", host[1]); break;
        case kCsrRowTooLong: snprintf(why, why_len, "a_row_offsets[i + 1] - a_row_offsets[i] > KSZ (i = %d)", host[1]); break;
        default: snprintf(why, why_len, "a_column_indices[i] >= KSZ or < 0 (i = %d)", host[1]); break;
        }
    }
    return DLSPM_ERR_CSR;
}

int dlspm_check_input(dlspm_ctx *ctx, int M, int K, int nnz, const int *row_offsets, const int *column_indices,
                      cudaStream_t st)
{
    if (!ctx->check_input || M <= 0 || !row_offsets) return DLSPM_OK;
    char why[160];
    const int rc = dlspm_sanity_check_csr(ctx, M, K, nnz, row_offsets, column_indices, why, sizeof(why), (void *)st);
    if (rc == DLSPM_ERR_CSR) snprintf(ctx->last_error, sizeof(ctx->last_error), "input check: %s", why);
    return rc;
}

int dlspm_check_input_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                           const int *column_indices)
{
    if (!ctx->check_input || M <= 0 || !row_offsets) return DLSPM_OK;
    char why[160];
    const int rc = dlspm_sanity_check_csr_host(M, K, N, nnz, row_offsets, column_indices, why, sizeof(why));
    if (rc != DLSPM_OK) snprintf(ctx->last_error, sizeof(ctx->last_error), "input check: %s", why);
    return rc;
}
