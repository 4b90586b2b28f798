// The benchmark's denominator: cuBLASLt bf16 GEMM on the same operands, configured
// as the reference configures it (experiments/src/cublaslt.rs:446-466):
// COMPUTE_32F with fp32 scale, C^ = (B^)^T . A^ in cuBLASLt's column-major
// terms -- first operand our `b` transposed, second our `a` -- layouts
// (k, n, k), (k, m, k), (n, m, n), bf16 output, 32 MiB workspace, first
// heuristic. Built into its own library, loaded by the benchmark only.
#include <cstdint>
#include <cstdio>
#include <cublasLt.h>
#include <cuda_runtime.h>

namespace {
constexpr size_t kWorkspaceBytes = 32u << 20;

struct Session {
    cublasLtHandle_t handle = nullptr;
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, d = nullptr;
    cublasLtMatmulPreference_t preference = nullptr;
    cublasLtMatmulHeuristicResult_t heuristic{};
    void* workspace = nullptr;
    uint32_t m = 0, n = 0, k = 0;
    bool ready = false;
};
Session session;
char error_text[256] = "";

int fail(const char* what, int status) {
    snprintf(error_text, sizeof error_text, "%s failed with status %d", what, status);
    return -1;
}
}  // namespace

extern "C" const char* fkb_last_error(void) { return error_text; }
extern "C" size_t fkb_version(void) { return cublasLtGetVersion(); }

extern "C" int fkb_prepare(uint32_t m, uint32_t n, uint32_t k) {
    if (session.ready && session.m == m && session.n == n && session.k == k) return 0;
    cublasStatus_t status;
    if (!session.handle && (status = cublasLtCreate(&session.handle)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtCreate", status);
    if (session.desc) cublasLtMatmulDescDestroy(session.desc);
    if (session.a) cublasLtMatrixLayoutDestroy(session.a);
    if (session.b) cublasLtMatrixLayoutDestroy(session.b);
    if (session.d) cublasLtMatrixLayoutDestroy(session.d);
    if (session.preference) cublasLtMatmulPreferenceDestroy(session.preference);
    session.ready = false;
    if ((status = cublasLtMatmulDescCreate(&session.desc, CUBLAS_COMPUTE_32F, CUDA_R_32F)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtMatmulDescCreate", status);
    const cublasOperation_t transposed = CUBLAS_OP_T, plain = CUBLAS_OP_N;
    cublasLtMatmulDescSetAttribute(session.desc, CUBLASLT_MATMUL_DESC_TRANSA, &transposed, sizeof transposed);
    cublasLtMatmulDescSetAttribute(session.desc, CUBLASLT_MATMUL_DESC_TRANSB, &plain, sizeof plain);
    if ((status = cublasLtMatrixLayoutCreate(&session.a, CUDA_R_16BF, k, n, k)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtMatrixLayoutCreate(a)", status);
    if ((status = cublasLtMatrixLayoutCreate(&session.b, CUDA_R_16BF, k, m, k)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtMatrixLayoutCreate(b)", status);
    if ((status = cublasLtMatrixLayoutCreate(&session.d, CUDA_R_16BF, n, m, n)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtMatrixLayoutCreate(d)", status);
    if ((status = cublasLtMatmulPreferenceCreate(&session.preference)) != CUBLAS_STATUS_SUCCESS)
        return fail("cublasLtMatmulPreferenceCreate", status);
    const size_t workspace = kWorkspaceBytes;
    cublasLtMatmulPreferenceSetAttribute(session.preference, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                         &workspace, sizeof workspace);
    int found = 0;
    status = cublasLtMatmulAlgoGetHeuristic(session.handle, session.desc, session.a, session.b, session.d,
                                            session.d, session.preference, 1, &session.heuristic, &found);
    if (status != CUBLAS_STATUS_SUCCESS || found == 0) return fail("cublasLtMatmulAlgoGetHeuristic", status);
    if (!session.workspace && cudaMalloc(&session.workspace, kWorkspaceBytes) != cudaSuccess)
        return fail("cudaMalloc(workspace)", 0);
    session.m = m;
    session.n = n;
    session.k = k;
    session.ready = true;
    return 0;
}

// C[m, n] = A[m, k] . B[n, k]^T with our row-major operand names.
extern "C" int fkb_gemm(const void* a, const void* b, void* c, void* stream) {
    if (!session.ready) return fail("fkb_gemm before fkb_prepare", 0);
    const float one = 1.0f, zero = 0.0f;
    const cublasStatus_t status = cublasLtMatmul(
        session.handle, session.desc, &one, b, session.a, a, session.b, &zero, c, session.d, c,
        session.d, &session.heuristic.algo, session.workspace, kWorkspaceBytes,
        static_cast<cudaStream_t>(stream));
    if (status != CUBLAS_STATUS_SUCCESS) return fail("cublasLtMatmul", status);
    return 0;
}
