// Entry points that take HOST buffers: copy in, run the device entry point, copy out.  These are the
// calls a program that keeps its matrices in host memory binds to, as the reference drivers do
// around their kernels (explicit memcpy before and after, SPMM/spmm-esimd-fromfile.cpp:172-180,255).
// Device staging memory belongs to the context and is reused between calls.  Pinned host memory
// makes the copies asynchronous DMA; pageable memory works too.
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace {

struct Carver {
    char *base;
    size_t off;
    explicit Carver(void *b) : base((char *)b), off(0) {}
    template <typename T>
    T *take(size_t n)
    {
        T *p = (T *)(base + off);
        off += (n * sizeof(T) + 255) & ~(size_t)255;
        return p;
    }
};

inline size_t padded(size_t bytes) { return (bytes + 255) & ~(size_t)255; }

// A host-buffer call that fails half-way may still have copies and kernels in flight that read the
// staging memory or write the caller's buffers.  Every such call therefore leaves through here: on
// an error the streams it used are drained before the error is reported, so that when the call
// returns nothing of it is running any more.
int drain_on_error(dlspm_ctx *ctx, int rc)
{
    if (rc == DLSPM_OK || !ctx) return rc;
    if (cudaSetDevice(ctx->device) == cudaSuccess) {
        if (ctx->stream) (void)cudaStreamSynchronize(ctx->stream);
        if (ctx->pipeline_ready) {
            (void)cudaStreamSynchronize(ctx->h2d_stream);
            (void)cudaStreamSynchronize(ctx->d2h_stream);
        }
    }
    (void)cudaGetLastError();
    return rc;
}

}  // namespace

static int dlspm_spmm_csr_f32_host_impl(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                                       const int *row_offsets, const int *column_indices, const float *B,
                                       float *C)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && (!values || !column_indices)) || ((size_t)K * N > 0 && !B) ||
        ((size_t)M * N > 0 && !C))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nB = (size_t)K * N, nC = (size_t)M * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + 2 * padded(4 * (size_t)nnz) + padded(4 * nB) +
                                      padded(4 * nC) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_v = cv.take<float>((size_t)nnz);
    float *d_B = cv.take<float>(nB);
    float *d_C = cv.take<float>(nC);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) {
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_v, values, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    }
    if (nB) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, B, 4 * nB, cudaMemcpyHostToDevice, st));
    rc = dlspm_spmm_csr_f32(ctx, M, K, N, nnz, d_v, d_ro, d_ci, d_B, d_C, st);
    if (rc) return rc;
    if (nC) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(C, d_C, 4 * nC, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

static int dlspm_sddmm_csr_f32_host_impl(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                                        const int *column_indices, const float *lhs, const float *rhs,
                                        float *out_values)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && (!column_indices || !out_values)) || ((size_t)M * N > 0 && !lhs) ||
        ((size_t)K * N > 0 && !rhs))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nL = (size_t)M * N, nR = (size_t)K * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + 2 * padded(4 * (size_t)nnz) + padded(4 * nL) +
                                      padded(4 * nR) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_out = cv.take<float>((size_t)nnz);
    float *d_L = cv.take<float>(nL);
    float *d_R = cv.take<float>(nR);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    if (nL) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_L, lhs, 4 * nL, cudaMemcpyHostToDevice, st));
    if (nR) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_R, rhs, 4 * nR, cudaMemcpyHostToDevice, st));
    rc = dlspm_sddmm_csr_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_L, d_R, d_out, st);
    if (rc) return rc;
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(out_values, d_out, 4 * (size_t)nnz, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

static int dlspm_fused_sddmm_spmm_f32_host_impl(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                               const int *row_offsets, const int *column_indices,
                                               const float *C, const float *B, const float *D, float *E)
{
    if (!ctx || M < 0 || K < 0 || N < 0 || nnz < 0) return DLSPM_ERR_INVALID_ARGUMENT;
    if (!row_offsets || (nnz > 0 && !column_indices) || ((size_t)M * N > 0 && (!C || !E)) ||
        ((size_t)K * N > 0 && (!B || !D)))
        return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t nM = (size_t)M * N, nK = (size_t)K * N;
    rc = dlspm_stage_reserve(ctx, padded(4 * ((size_t)M + 1)) + padded(4 * (size_t)nnz) + 2 * padded(4 * nM) +
                                      2 * padded(4 * nK) + 256);
    if (rc) return rc;
    Carver cv(ctx->stage);
    int *d_ro = cv.take<int>((size_t)M + 1);
    int *d_ci = cv.take<int>((size_t)nnz);
    float *d_C = cv.take<float>(nM);
    float *d_E = cv.take<float>(nM);
    float *d_B = cv.take<float>(nK);
    float *d_D = cv.take<float>(nK);
    cudaStream_t st = ctx->stream;
    DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ro, row_offsets, 4 * ((size_t)M + 1), cudaMemcpyHostToDevice, st));
    if (nnz) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_ci, column_indices, 4 * (size_t)nnz, cudaMemcpyHostToDevice, st));
    if (nM) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_C, C, 4 * nM, cudaMemcpyHostToDevice, st));
    if (nK) {
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_B, B, 4 * nK, cudaMemcpyHostToDevice, st));
        DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(d_D, D, 4 * nK, cudaMemcpyHostToDevice, st));
    }
    rc = dlspm_fused_sddmm_spmm_f32(ctx, M, K, N, nnz, d_ro, d_ci, d_C, d_B, d_D, d_E, st);
    if (rc) return rc;
    if (nM) DLSPM_CUDA_TRY(ctx, cudaMemcpyAsync(E, d_E, 4 * nM, cudaMemcpyDeviceToHost, st));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return DLSPM_OK;
}

// Batched SpMM with host pointers, pipelined: the batch is cut into pieces of at most 128 MiB of
// device copies; kPipeSlots staging buffers rotate, and three streams overlap the host-to-device
// copies of the next pieces, the grouped launch of the current one and the device-to-host copies
// of the previous ones (PCIe is full duplex, so the slower of the two copy directions bounds the
// call, not their sum).  More than two slots keep the inbound copies running while a finished
// piece still waits for its turn on the outbound stream.
namespace {

// Copies between host and device arrays that merge neighbours into one cudaMemcpyAsync.  Two arrays
// are neighbours when the distance between their host addresses equals the distance between their
// device addresses (the staging layout packs arrays at 256-byte boundaries in call order) and both
// lie in ONE host allocation known to the driver (one cudaHostAlloc / cudaHostRegister range), so
// that the few padding bytes between them are readable and the whole run is pinned.  A caller that
// keeps its batch in one pinned arena in the staging order (per problem: row_offsets,
// column_indices, values, B, each padded to 256 bytes; results likewise in a second arena) gets one
// copy per 128 MiB piece and direction; any other layout is copied array by array as before.
class RunCopier {
public:
    RunCopier(dlspm_ctx *ctx, cudaStream_t st, bool to_device) : ctx_(ctx), st_(st), to_device_(to_device) {}

    int add(void *dev, const void *host, size_t bytes)
    {
        if (bytes == 0) return DLSPM_OK;
        char *d = (char *)dev;
        const char *h = (const char *)host;
        if (run_bytes_ && d >= run_d_ + run_bytes_ && (size_t)(d - (run_d_ + run_bytes_)) < 256 &&
            h == run_h_ + (d - run_d_) && same_host_range(run_h_, h + bytes)) {
            run_bytes_ = (size_t)(d - run_d_) + bytes;
            return DLSPM_OK;
        }
        int rc = flush();
        if (rc) return rc;
        run_d_ = d;
        run_h_ = h;
        run_bytes_ = bytes;
        return DLSPM_OK;
    }

    int flush()
    {
        if (!run_bytes_) return DLSPM_OK;
        const size_t n = run_bytes_;
        run_bytes_ = 0;
        copies_++;
        if (to_device_) DLSPM_CUDA_TRY(ctx_, cudaMemcpyAsync(run_d_, run_h_, n, cudaMemcpyHostToDevice, st_));
        else DLSPM_CUDA_TRY(ctx_, cudaMemcpyAsync(const_cast<char *>(run_h_), run_d_, n, cudaMemcpyDeviceToHost, st_));
        return DLSPM_OK;
    }

    long long copies() const { return copies_; }

private:
    // CUresult cuPointerGetAttribute(void *data, CUpointer_attribute attribute, CUdeviceptr ptr)
    typedef int (*PtrAttrFn)(void *, int, unsigned long long);

    static PtrAttrFn driver_query()
    {
        static PtrAttrFn fn = []() -> PtrAttrFn {
            void *p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &p, cudaEnableDefault, &q) != cudaSuccess ||
                q != cudaDriverEntryPointSuccess) {
                (void)cudaGetLastError();
                return nullptr;
            }
            return (PtrAttrFn)p;
        }();
        return fn;
    }

    // true when [a, b) lies inside one host allocation registered with the driver
    bool same_host_range(const char *a, const char *b)
    {
        if (a >= range_lo_ && b <= range_hi_) return true;
        PtrAttrFn fn = driver_query();
        if (!fn) return false;
        unsigned long long start = 0;
        size_t size = 0;
        const int kRangeStart = 11, kRangeSize = 12;  // CU_POINTER_ATTRIBUTE_RANGE_START_ADDR / _RANGE_SIZE
        if (fn(&start, kRangeStart, (unsigned long long)(uintptr_t)a) != 0 ||
            fn(&size, kRangeSize, (unsigned long long)(uintptr_t)a) != 0)
            return false;  // pageable or unknown memory: never merged
        range_lo_ = (const char *)(uintptr_t)start;
        range_hi_ = range_lo_ + size;
        return a >= range_lo_ && b <= range_hi_;
    }

    dlspm_ctx *ctx_;
    cudaStream_t st_;
    bool to_device_;
    char *run_d_ = nullptr;
    const char *run_h_ = nullptr;
    size_t run_bytes_ = 0;
    const char *range_lo_ = nullptr, *range_hi_ = nullptr;
    long long copies_ = 0;
};

int pipeline_init(dlspm_ctx *ctx)
{
    if (ctx->pipeline_ready) return DLSPM_OK;
    DLSPM_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
    DLSPM_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    for (int i = 0; i < kPipeSlots; i++) {
        DLSPM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_h2d[i], cudaEventDisableTiming));
        DLSPM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_kernel[i], cudaEventDisableTiming));
        DLSPM_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_d2h[i], cudaEventDisableTiming));
    }
    ctx->pipeline_ready = 1;
    return DLSPM_OK;
}

}  // namespace

static int dlspm_spmm_batched_f32_host_impl(dlspm_ctx *ctx, int count, const dlspm_problem *problems)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    const size_t budget = (size_t)128 << 20;
    auto need = [](const dlspm_problem &q) {
        return padded(4 * ((size_t)q.M + 1)) + 2 * padded(4 * (size_t)q.nnz) + padded(4 * (size_t)q.K * q.N) +
               padded(4 * (size_t)q.M * q.N);
    };
    size_t largest = 0;
    for (int i = 0; i < count; i++) {
        const dlspm_problem &q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || q.nnz < 0 || !q.row_offsets ||
            (q.nnz > 0 && (!q.values || !q.column_indices)) || ((size_t)q.K * q.N > 0 && !q.B) ||
            ((size_t)q.M * q.N > 0 && !q.C))
            return DLSPM_ERR_INVALID_ARGUMENT;
        rc = dlspm_check_input_host(ctx, q.M, q.K, q.N, q.nnz, q.row_offsets, q.column_indices);  // DLSPM_OPT_CHECK_INPUT
        if (rc) return rc;
        largest = std::max(largest, need(q));
    }
    if (count == 0) return DLSPM_OK;
    rc = pipeline_init(ctx);
    if (rc) return rc;
    // pieces: consecutive problems up to the budget (a single larger problem is its own piece)
    std::vector<int> piece_end;
    size_t max_piece = 0, max_tables = 0;
    for (int first = 0; first < count;) {
        size_t bytes = 0;
        int last = first;
        while (last < count && (last == first || bytes + need(problems[last]) <= budget)) bytes += need(problems[last++]);
        piece_end.push_back(last);
        max_piece = std::max(max_piece, bytes);
        max_tables = std::max(max_tables, dlspm_batched_table_bytes(last - first));
        first = last;
    }
    const size_t slot = padded(max_piece) + padded(max_tables);
    rc = dlspm_stage_reserve(ctx, (size_t)kPipeSlots * slot + 256);
    if (rc) return rc;
    // the launch tables travel from pinned memory: a copy from pageable memory would synchronise
    // the compute stream with the host and serialise the pipeline
    if (ctx->pinned_bytes < (size_t)kPipeSlots * padded(max_tables)) {
        if (ctx->pinned) cudaFreeHost(ctx->pinned);
        ctx->pinned = nullptr;
        ctx->pinned_bytes = 0;
        cudaError_t perr = cudaMallocHost(&ctx->pinned, (size_t)kPipeSlots * padded(max_tables));
        if (perr != cudaSuccess) {
            dlspm_cuda_fail(ctx, perr, "cudaMallocHost(tables)");
            return DLSPM_ERR_NOMEM;
        }
        ctx->pinned_bytes = (size_t)kPipeSlots * padded(max_tables);
    }
    cudaStream_t h2d = ctx->h2d_stream, run = ctx->stream, d2h = ctx->d2h_stream;
    std::vector<dlspm_problem> dev[kPipeSlots];
    int first = 0;
    for (size_t pi = 0; pi < piece_end.size(); pi++) {
        const int last = piece_end[pi];
        const int b = (int)(pi % kPipeSlots);
        char *base = (char *)ctx->stage + (size_t)b * slot;
        // the slot is free once the results of the piece that used it last have left; its pinned
        // table may be rewritten once that piece's launch has finished
        if (pi >= (size_t)kPipeSlots) {
            DLSPM_CUDA_TRY(ctx, cudaStreamWaitEvent(h2d, ctx->ev_d2h[b], 0));
            DLSPM_CUDA_TRY(ctx, cudaEventSynchronize(ctx->ev_kernel[b]));
        }
        // staging layout of a piece: the inputs of all its problems first (per problem row_offsets,
        // column_indices, values, B), then all results, every array at a 256-byte boundary
        Carver cv(base + padded(max_tables));
        dev[b].clear();
        RunCopier in(ctx, h2d, true);
        for (int i = first; i < last; i++) {
            const dlspm_problem &q = problems[i];
            dlspm_problem d = q;
            int *d_ro = cv.take<int>((size_t)q.M + 1);
            int *d_ci = cv.take<int>((size_t)q.nnz);
            float *d_v = cv.take<float>((size_t)q.nnz);
            float *d_B = cv.take<float>((size_t)q.K * q.N);
            rc = in.add(d_ro, q.row_offsets, 4 * ((size_t)q.M + 1));
            if (!rc) rc = in.add(d_ci, q.column_indices, 4 * (size_t)q.nnz);
            if (!rc) rc = in.add(d_v, q.values, 4 * (size_t)q.nnz);
            if (!rc) rc = in.add(d_B, q.B, 4 * (size_t)q.K * q.N);
            if (rc) return rc;
            d.row_offsets = d_ro;
            d.column_indices = d_ci;
            d.values = d_v;
            d.B = d_B;
            dev[b].push_back(d);
        }
        rc = in.flush();
        if (rc) return rc;
        for (int i = first; i < last; i++) {
            const dlspm_problem &q = problems[i];
            dev[b][(size_t)(i - first)].C = cv.take<float>((size_t)q.M * q.N);
        }
        ctx->host_copies += in.copies();
        DLSPM_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_h2d[b], h2d));
        DLSPM_CUDA_TRY(ctx, cudaStreamWaitEvent(run, ctx->ev_h2d[b], 0));
        rc = dlspm_spmm_batched_at(ctx, (int)dev[b].size(), dev[b].data(), base, run,
                                   (char *)ctx->pinned + (size_t)b * padded(max_tables));
        if (rc) return rc;
        DLSPM_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_kernel[b], run));
        DLSPM_CUDA_TRY(ctx, cudaStreamWaitEvent(d2h, ctx->ev_kernel[b], 0));
        RunCopier outc(ctx, d2h, false);
        for (int i = first; i < last; i++) {
            const dlspm_problem &q = problems[i];
            rc = outc.add(dev[b][(size_t)(i - first)].C, q.C, 4 * (size_t)q.M * q.N);
            if (rc) return rc;
        }
        rc = outc.flush();
        if (rc) return rc;
        ctx->host_copies += outc.copies();
        DLSPM_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_d2h[b], d2h));
        first = last;
    }
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(d2h));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(run));
    DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(h2d));
    return DLSPM_OK;
}

// ---- grouped SDDMM and fused chain with host pointers ---------------------------------------------
// Pieces of up to 256 MiB of device copies, one after the other on the context's stream: inputs in
// (merged into few copies where the caller's arrays are neighbours in one pinned allocation), one
// grouped launch, results out.
namespace {

struct SddmmTraits {
    typedef dlspm_sddmm_problem Problem;
    static bool valid(const Problem &q)
    {
        return q.M >= 0 && q.K >= 0 && q.N >= 0 && q.nnz >= 0 && q.row_offsets &&
               (q.nnz == 0 || (q.column_indices && q.out_values)) && ((size_t)q.M * q.N == 0 || q.lhs) &&
               ((size_t)q.K * q.N == 0 || q.rhs);
    }
    static size_t need(const Problem &q)
    {
        return padded(4 * ((size_t)q.M + 1)) + 3 * padded(4 * (size_t)q.nnz) + padded(4 * (size_t)q.M * q.N) +
               padded(4 * (size_t)q.K * q.N);
    }
    // carves the device arrays of one problem, queues its input copies, returns the device problem
    static int stage(RunCopier &in, Carver &cv, const Problem &q, Problem &d)
    {
        d = q;
        int *ro = cv.take<int>((size_t)q.M + 1);
        int *ci = cv.take<int>((size_t)q.nnz);
        float *mask = q.mask_values ? cv.take<float>((size_t)q.nnz) : nullptr;
        float *lhs = cv.take<float>((size_t)q.M * q.N);
        float *rhs = cv.take<float>((size_t)q.K * q.N);
        int rc = in.add(ro, q.row_offsets, 4 * ((size_t)q.M + 1));
        if (!rc) rc = in.add(ci, q.column_indices, 4 * (size_t)q.nnz);
        if (!rc && mask) rc = in.add(mask, q.mask_values, 4 * (size_t)q.nnz);
        if (!rc) rc = in.add(lhs, q.lhs, 4 * (size_t)q.M * q.N);
        if (!rc) rc = in.add(rhs, q.rhs, 4 * (size_t)q.K * q.N);
        d.row_offsets = ro;
        d.column_indices = ci;
        d.mask_values = mask;
        d.lhs = lhs;
        d.rhs = rhs;
        return rc;
    }
    static void carve_out(Carver &cv, const Problem &q, Problem &d) { d.out_values = cv.take<float>((size_t)q.nnz); }
    static int unstage(RunCopier &out, const Problem &q, const Problem &d) { return out.add(d.out_values, q.out_values, 4 * (size_t)q.nnz); }
    static int run(dlspm_ctx *ctx, int n, const Problem *d, void *tables, cudaStream_t st) { return dlspm_sddmm_batched_at(ctx, n, d, tables, nullptr, st); }
};

struct FusedTraits {
    typedef dlspm_fused_problem Problem;
    static bool valid(const Problem &q)
    {
        return q.M >= 0 && q.K >= 0 && q.N >= 0 && q.nnz >= 0 && q.row_offsets && (q.nnz == 0 || q.column_indices) &&
               ((size_t)q.M * q.N == 0 || (q.C && q.E)) && ((size_t)q.K * q.N == 0 || (q.B && q.D));
    }
    static size_t need(const Problem &q)
    {
        return padded(4 * ((size_t)q.M + 1)) + padded(4 * (size_t)q.nnz) + 2 * padded(4 * (size_t)q.M * q.N) +
               2 * padded(4 * (size_t)q.K * q.N);
    }
    static int stage(RunCopier &in, Carver &cv, const Problem &q, Problem &d)
    {
        d = q;
        int *ro = cv.take<int>((size_t)q.M + 1);
        int *ci = cv.take<int>((size_t)q.nnz);
        float *c = cv.take<float>((size_t)q.M * q.N);
        float *b = cv.take<float>((size_t)q.K * q.N);
        float *dd = cv.take<float>((size_t)q.K * q.N);
        int rc = in.add(ro, q.row_offsets, 4 * ((size_t)q.M + 1));
        if (!rc) rc = in.add(ci, q.column_indices, 4 * (size_t)q.nnz);
        if (!rc) rc = in.add(c, q.C, 4 * (size_t)q.M * q.N);
        if (!rc) rc = in.add(b, q.B, 4 * (size_t)q.K * q.N);
        if (!rc) rc = in.add(dd, q.D, 4 * (size_t)q.K * q.N);
        d.row_offsets = ro;
        d.column_indices = ci;
        d.C = c;
        d.B = b;
        d.D = dd;
        return rc;
    }
    static void carve_out(Carver &cv, const Problem &q, Problem &d) { d.E = cv.take<float>((size_t)q.M * q.N); }
    static int unstage(RunCopier &out, const Problem &q, const Problem &d) { return out.add(d.E, q.E, 4 * (size_t)q.M * q.N); }
    static int run(dlspm_ctx *ctx, int n, const Problem *d, void *tables, cudaStream_t st) { return dlspm_fused_batched_at(ctx, n, d, tables, nullptr, st); }
};

template <typename T>
int rows_batched_host(dlspm_ctx *ctx, int count, const typename T::Problem *problems)
{
    if (!ctx || count < 0 || (count > 0 && !problems)) return DLSPM_ERR_INVALID_ARGUMENT;
    int rc = dlspm_use(ctx);
    if (rc) return rc;
    for (int i = 0; i < count; i++) {
        if (!T::valid(problems[i])) return DLSPM_ERR_INVALID_ARGUMENT;
        rc = dlspm_check_input_host(ctx, problems[i].M, problems[i].K, problems[i].N, problems[i].nnz,
                                    problems[i].row_offsets, problems[i].column_indices);  // DLSPM_OPT_CHECK_INPUT
        if (rc) return rc;
    }
    if (count == 0) return DLSPM_OK;
    const size_t budget = (size_t)256 << 20;
    std::vector<int> piece_end;
    size_t max_piece = 0, max_tables = 0;
    for (int first = 0; first < count;) {
        size_t bytes = 0;
        int last = first;
        while (last < count && (last == first || bytes + T::need(problems[last]) <= budget)) bytes += T::need(problems[last++]);
        piece_end.push_back(last);
        max_piece = std::max(max_piece, bytes);
        max_tables = std::max(max_tables, dlspm_rows_batched_table_bytes(last - first));
        first = last;
    }
    rc = dlspm_stage_reserve(ctx, padded(max_tables) + padded(max_piece) + 256);
    if (rc) return rc;
    cudaStream_t st = ctx->stream;
    std::vector<typename T::Problem> dev;
    int first = 0;
    for (int last : piece_end) {
        Carver cv((char *)ctx->stage + padded(max_tables));
        dev.assign((size_t)(last - first), typename T::Problem());
        RunCopier in(ctx, st, true);
        for (int i = first; i < last; i++) {
            rc = T::stage(in, cv, problems[i], dev[(size_t)(i - first)]);
            if (rc) return rc;
        }
        rc = in.flush();
        if (rc) return rc;
        for (int i = first; i < last; i++) T::carve_out(cv, problems[i], dev[(size_t)(i - first)]);
        rc = T::run(ctx, last - first, dev.data(), ctx->stage, st);
        if (rc) return rc;
        RunCopier out(ctx, st, false);
        for (int i = first; i < last; i++) {
            rc = T::unstage(out, problems[i], dev[(size_t)(i - first)]);
            if (rc) return rc;
        }
        rc = out.flush();
        if (rc) return rc;
        // the staging memory is reused by the next piece
        DLSPM_CUDA_TRY(ctx, cudaStreamSynchronize(st));
        first = last;
    }
    return DLSPM_OK;
}

}  // namespace

extern "C" int dlspm_sddmm_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_sddmm_problem *problems)
{
    return drain_on_error(ctx, rows_batched_host<SddmmTraits>(ctx, count, problems));
}

extern "C" int dlspm_fused_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_fused_problem *problems)
{
    return drain_on_error(ctx, rows_batched_host<FusedTraits>(ctx, count, problems));
}

// ---- exported entry points: the implementations above plus the drain on failure ---------------------
extern "C" int dlspm_spmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const float *values,
                                       const int *row_offsets, const int *column_indices, const float *B,
                                       float *C)
{
    return drain_on_error(ctx, dlspm_spmm_csr_f32_host_impl(ctx, M, K, N, nnz, values, row_offsets, column_indices, B, C));
}

extern "C" int dlspm_sddmm_csr_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz, const int *row_offsets,
                                        const int *column_indices, const float *lhs, const float *rhs,
                                        float *out_values)
{
    return drain_on_error(ctx, dlspm_sddmm_csr_f32_host_impl(ctx, M, K, N, nnz, row_offsets, column_indices, lhs, rhs, out_values));
}

extern "C" int dlspm_fused_sddmm_spmm_f32_host(dlspm_ctx *ctx, int M, int K, int N, int nnz,
                                               const int *row_offsets, const int *column_indices,
                                               const float *C, const float *B, const float *D, float *E)
{
    return drain_on_error(ctx, dlspm_fused_sddmm_spmm_f32_host_impl(ctx, M, K, N, nnz, row_offsets, column_indices, C, B, D, E));
}

extern "C" int dlspm_spmm_batched_f32_host(dlspm_ctx *ctx, int count, const dlspm_problem *problems)
{
    return drain_on_error(ctx, dlspm_spmm_batched_f32_host_impl(ctx, count, problems));
}

extern "C" int dlspm_host_copy_count(const dlspm_ctx *ctx, long long *copies)
{
    if (!ctx || !copies) return DLSPM_ERR_INVALID_ARGUMENT;
    *copies = ctx->host_copies;
    return DLSPM_OK;
}
