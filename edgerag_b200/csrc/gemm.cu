// Linear layers as library matrix products: out[M, N] = a[M, K] * w[N, K]^T through cuBLASLt.
//
// The reference's engine runs its projections through a library too (nn.Linear, cuBLAS), so the
// plain products stay with the library here; this file only pins down types and precision:
//   * float build:    every operand float, CUBLAS_COMPUTE_32F (no TF32, no reduced-precision mode)
//   * bfloat16 build: operands bfloat16, float accumulation, output bfloat16 or float
// Matrices are row-major with explicit leading dimensions.  The caller provides the workspace, so
// a call allocates nothing and can be captured in a CUDA graph.  Heuristic results are cached per
// shape.
#include <cublasLt.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
  size_t workspace = 0;
};

using Key = std::tuple<int, int, int, int, int, int, int, int, size_t>;

cublasLtHandle_t g_handle = nullptr;
std::map<Key, Plan> g_plans;
std::mutex g_mutex;

const char* status_name(cublasStatus_t s) {
  switch (s) {
    case CUBLAS_STATUS_SUCCESS: return "success";
    case CUBLAS_STATUS_NOT_INITIALIZED: return "not initialized";
    case CUBLAS_STATUS_ALLOC_FAILED: return "alloc failed";
    case CUBLAS_STATUS_INVALID_VALUE: return "invalid value";
    case CUBLAS_STATUS_ARCH_MISMATCH: return "arch mismatch";
    case CUBLAS_STATUS_EXECUTION_FAILED: return "execution failed";
    case CUBLAS_STATUS_INTERNAL_ERROR: return "internal error";
    case CUBLAS_STATUS_NOT_SUPPORTED: return "not supported";
    default: return "other";
  }
}

#define LT_CHECK(expr)                                                                         \
  do {                                                                                         \
    cublasStatus_t st__ = (expr);                                                              \
    if (st__ != CUBLAS_STATUS_SUCCESS)                                                         \
      return fail(ERB_ERR_CUDA, "linear: %s -> %s", #expr, status_name(st__));                 \
  } while (0)

int make_plan(Plan& p, int M, int N, int K, int lda, int ldw, int ldo, int out_f32, int accumulate,
              size_t ws_bytes) {
#if ERB_ELEM == 0
  const cudaDataType_t in_t = CUDA_R_32F;
  const cudaDataType_t out_t = CUDA_R_32F;
  if (!out_f32) return fail(ERB_ERR_ARG, "linear: the float build writes float only");
#else
  const cudaDataType_t in_t = CUDA_R_16BF;
  const cudaDataType_t out_t = out_f32 ? CUDA_R_32F : CUDA_R_16BF;
#endif
  (void)accumulate;
  LT_CHECK(cublasLtMatmulDescCreate(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
  const cublasOperation_t tt = CUBLAS_OP_T, nn = CUBLAS_OP_N;
  LT_CHECK(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &tt, sizeof(tt)));
  LT_CHECK(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &nn, sizeof(nn)));
  // Column-major view: C (N x M) = W^T-view (K x N, ld ldw)^T * a-view (K x M, ld lda).
  LT_CHECK(cublasLtMatrixLayoutCreate(&p.a, in_t, K, N, ldw));
  LT_CHECK(cublasLtMatrixLayoutCreate(&p.b, in_t, K, M, lda));
  LT_CHECK(cublasLtMatrixLayoutCreate(&p.c, out_t, N, M, ldo));
  cublasLtMatmulPreference_t pref;
  LT_CHECK(cublasLtMatmulPreferenceCreate(&pref));
  LT_CHECK(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes,
                                                sizeof(ws_bytes)));
  cublasLtMatmulHeuristicResult_t result;
  int found = 0;
  cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(g_handle, p.op, p.a, p.b, p.c, p.c, pref, 1, &result, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found == 0)
    return fail(ERB_ERR_UNSUPPORTED, "linear: no cuBLASLt algorithm for M=%d N=%d K=%d lda=%d ldw=%d ldo=%d (%s)",
                M, N, K, lda, ldw, ldo, status_name(st));
  p.algo = result.algo;
  p.workspace = result.workspaceSize;
  return ERB_OK;
}

}  // namespace

// out[M, N] (+)= a[M, K] * w[N, K]^T.  `out_f32` selects a float output in the bfloat16 build;
// `accumulate` adds to what `out` holds (beta = 1) instead of overwriting it.
ERB_EXPORT int erb_linear(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw,
                          int ldo, int out_f32, int accumulate, void* workspace, long long ws_bytes,
                          void* stream) {
  if (M <= 0) return ERB_OK;
  if (N <= 0 || K <= 0 || lda < K || ldw < K || ldo < N) return fail(ERB_ERR_ARG, "linear: bad sizes");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_handle) LT_CHECK(cublasLtCreate(&g_handle));
  const size_t ws = workspace ? (size_t)ws_bytes : 0;
  Key key{M, N, K, lda, ldw, ldo, out_f32, accumulate, ws};
  auto it = g_plans.find(key);
  if (it == g_plans.end()) {
    Plan p;
    int rc = make_plan(p, M, N, K, lda, ldw, ldo, out_f32, accumulate, ws);
    if (rc) return rc;
    it = g_plans.emplace(key, p).first;
  }
  const Plan& p = it->second;
  const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
  LT_CHECK(cublasLtMatmul(g_handle, p.op, &alpha, w, p.a, a, p.b, &beta, out, p.c, out, p.c, &p.algo,
                          workspace, ws, (cudaStream_t)stream));
  return ERB_OK;
}

#if ERB_ELEM == 1
// ---------------------------------------------------------------------------------------------
// Weight-streaming product for a handful of rows (decode): out[M, N] = a[M, K] * w[N, K]^T with
// M <= 16, bfloat16 operands, float accumulation.  The work is reading w once at memory speed:
// each warp owns two rows of w and walks K with 16-byte loads, eight chunks per row in flight
// before any is used; the few rows of `a` are re-read from L1.  Sums are reduced over the warp
// in a fixed order, so the result does not depend on the launch geometry.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kSkWarps = 8;
constexpr int kSkRows = 2;       // rows of w per warp
constexpr int kSkUnroll = 4;     // 16-byte chunks per row and lane in flight

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int MT, bool OUT_F32>
__global__ void __launch_bounds__(kSkWarps * 32)
linear_skinny_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                     int M, int N, int K, int lda, int ldw, int ldo) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kSkWarps + warp) * kSkRows;
  if (n0 >= N) return;
  float acc[MT][kSkRows];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int r = 0; r < kSkRows; ++r) acc[m][r] = 0.f;
  const __nv_bfloat16* wr[kSkRows];
#pragma unroll
  for (int r = 0; r < kSkRows; ++r) wr[r] = w + (size_t)min(n0 + r, N - 1) * ldw;

  const int chunks = K >> 3;                     // 16-byte chunks per row
  for (int c0 = lane; c0 < chunks; c0 += 32 * kSkUnroll) {
    uint4 raw[kSkRows][kSkUnroll];
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {
      const int c = c0 + 32 * u;
#pragma unroll
      for (int r = 0; r < kSkRows; ++r)
        raw[r][u] = (c < chunks) ? __ldcs(reinterpret_cast<const uint4*>(wr[r]) + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {
      const int c = c0 + 32 * u;
      if (c >= chunks) break;
      float wf[kSkRows][8];
#pragma unroll
      for (int r = 0; r < kSkRows; ++r) unpack_bf16x8(raw[r][u], wf[r]);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          float xf[8];
          unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(a + (size_t)m * lda) + c), xf);
#pragma unroll
          for (int r = 0; r < kSkRows; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[m][r] = fmaf(xf[i], wf[r][i], acc[m][r]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int r = 0; r < kSkRows; ++r) acc[m][r] = warp_sum(acc[m][r]);
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= M) break;
#pragma unroll
      for (int r = 0; r < kSkRows; ++r) {
        if (n0 + r < N) {
          if (OUT_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n0 + r] = acc[m][r];
          else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n0 + r] = __float2bfloat16_rn(acc[m][r]);
        }
      }
    }
  }
}

template <int MT>
int launch_skinny(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldo,
                  int out_f32, cudaStream_t s) {
  const int rows_per_block = kSkWarps * kSkRows;
  const unsigned blocks = (unsigned)((N + rows_per_block - 1) / rows_per_block);
  if (out_f32)
    linear_skinny_kernel<MT, true><<<blocks, kSkWarps * 32, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                                     out, M, N, K, lda, ldw, ldo);
  else
    linear_skinny_kernel<MT, false><<<blocks, kSkWarps * 32, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                                      out, M, N, K, lda, ldw, ldo);
  return check_launch("linear_skinny");
}

}  // namespace

// Same result contract as erb_linear (no accumulate), for 1 <= M <= 16 with K, lda and ldw
// multiples of 8 elements and 16-byte aligned operands.
ERB_EXPORT int erb_linear_skinny(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw,
                                 int ldo, int out_f32, void* stream) {
  if (M <= 0) return ERB_OK;
  if (M > 16) return fail(ERB_ERR_UNSUPPORTED, "linear_skinny: %d rows (at most 16)", M);
  if (N <= 0 || K <= 0 || lda < K || ldw < K || ldo < N) return fail(ERB_ERR_ARG, "linear_skinny: bad sizes");
  if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return fail(ERB_ERR_UNSUPPORTED, "linear_skinny: K and the leading dimensions must be multiples of 8");
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 2) return launch_skinny<2>(a, w, out, M, N, K, lda, ldw, ldo, out_f32, s);
  if (M <= 4) return launch_skinny<4>(a, w, out, M, N, K, lda, ldw, ldo, out_f32, s);
  if (M <= 8) return launch_skinny<8>(a, w, out, M, N, K, lda, ldw, ldo, out_f32, s);
  return launch_skinny<16>(a, w, out, M, N, K, lda, ldw, ldo, out_f32, s);
}
#endif  // ERB_ELEM == 1
