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
  // other algorithms the library proposed for this shape (the first is its own first choice), to be
  // timed against each other on the first call that is not inside a stream capture
  cublasLtMatmulHeuristicResult_t candidates[8];
  int n_candidates = 0;
  bool tuned = false;
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

int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return (v && v[0]) ? atoi(v) : fallback;
}

bool tuning_enabled() {
  static const bool on = [] {
    const char* v = getenv("EDGERAG_B200_NO_TUNE");
    return !(v && v[0] == '1');
  }();
  return on;
}

// The library's first choice is not always its fastest algorithm for a shape (the products of a 2,048-token
// portion: 5 % of the step).  A trial of a layer's four shapes costs as much as several steps, so it is for
// shapes that keep coming back, and the caller knows which those are: it switches trials on (erb_linear_tune)
// around a run whose shapes it expects to use many times more (the engine: the run before a step's layout is
// captured into a CUDA graph, which happens when the layout is seen a second time and fixes the algorithms
// for every replay).  During such a run, outside a stream capture, every proposal for a shape of 1,024 rows
// or more runs a few times on the caller's operands (each writes the same product to `out`), every run after
// a write of more than L2's size so that the weights come from DRAM as they do in a step, timed with events;
// a proposal's fastest of three runs counts, one that is 15 % behind the best so far gets no further runs,
// and the fastest proposal stays: one choice per shape and process.  Not below 1,024 rows: for the 17 to
// 64 rows of a decode step none of the proposals beat the first, and when the 513 to 576 rows of serving
// steps were tried (then with the weights in L2) the choices were slower inside the step.
constexpr int kTuneFromRows = 1024;
bool g_tune_now = false;         // set by the caller around a run whose shapes are worth a trial (erb_linear_tune)
int g_trials = 0;                // trials run so far in this process
constexpr size_t kFlushBytes = 192u << 20;

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
  int found = 0;
  const int want = (M >= kTuneFromRows && tuning_enabled()) ? 8 : 1;   // more than one only where they get timed
  cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(g_handle, p.op, p.a, p.b, p.c, p.c, pref, want, p.candidates, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found == 0)
    return fail(ERB_ERR_UNSUPPORTED, "linear: no cuBLASLt algorithm for M=%d N=%d K=%d lda=%d ldw=%d ldo=%d (%s)",
                M, N, K, lda, ldw, ldo, status_name(st));
  p.n_candidates = found;
  p.algo = p.candidates[0].algo;
  p.workspace = p.candidates[0].workspaceSize;
  return ERB_OK;
}

void tune_plan(Plan& p, int M, int N, int K, const void* a, const void* w, void* out, void* workspace, size_t ws, cudaStream_t stream) {
  if (p.n_candidates < 2 || M < kTuneFromRows || !tuning_enabled()) { p.tuned = true; return; }
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) return;
  if (!g_tune_now) return;
  p.tuned = true;
  ++g_trials;
  const bool log = env_int("EDGERAG_B200_TUNE_LOG", 0) != 0;
  // In a step the weights of a product come from DRAM (a layer's weights pass through L2 long before
  // the layer runs again), so every timed run starts after a buffer larger than L2 has been written.
  void* flush = nullptr;
  if (cudaMalloc(&flush, kFlushBytes) != cudaSuccess) { cudaGetLastError(); return; }
  cudaEvent_t t0, t1;
  if (cudaEventCreate(&t0) != cudaSuccess) { cudaFree(flush); return; }
  if (cudaEventCreate(&t1) != cudaSuccess) { cudaEventDestroy(t0); cudaFree(flush); return; }
  const float alpha = 1.f, beta = 0.f;
  float best = 1e30f;
  int best_i = 0;
  for (int i = 0; i < p.n_candidates; ++i) {
    const cublasLtMatmulHeuristicResult_t& c = p.candidates[i];
    if (c.state != CUBLAS_STATUS_SUCCESS || c.workspaceSize > ws) continue;
    bool ok = true;
    float fastest = 1e30f;
    for (int r = 0; r < 4 && ok; ++r) {     // one to warm up, three timed: the fastest counts (what disturbs a run only adds)
      cudaMemsetAsync(flush, r, kFlushBytes, stream);
      cudaEventRecord(t0, stream);
      ok = cublasLtMatmul(g_handle, p.op, &alpha, w, p.a, a, p.b, &beta, out, p.c, out, p.c, &c.algo, workspace, ws,
                          stream) == CUBLAS_STATUS_SUCCESS;
      cudaEventRecord(t1, stream);
      float ms = 0.f;
      ok = ok && cudaEventSynchronize(t1) == cudaSuccess && cudaEventElapsedTime(&ms, t0, t1) == cudaSuccess;
      if (r && ms < fastest) fastest = ms;
      if (r && ms > 1.15f * best) break;    // (no match for the best so far: its other runs are saved)
    }
    if (!ok) { cudaGetLastError(); continue; }
    if (log) fprintf(stderr, "[edgerag_b200] linear %d x %d x %d: proposal %d, %.1f us\n", M, N, K, i, fastest * 1000);
    if (fastest < best) { best = fastest; best_i = i; }
  }
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(flush);
  p.algo = p.candidates[best_i].algo;
  p.workspace = p.candidates[best_i].workspaceSize;
}

}  // namespace

// Trials of the library's proposals (see tune_plan) on or off for the products that follow.
ERB_EXPORT int erb_linear_tune(int on) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_tune_now = on != 0;
  return ERB_OK;
}

// How many shapes have had a trial in this process.
ERB_EXPORT int erb_linear_trials() {
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_trials;
}

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
  Plan& p = it->second;
  if (!p.tuned && !accumulate) tune_plan(p, M, N, K, a, w, out, workspace, ws, (cudaStream_t)stream);
  const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
  LT_CHECK(cublasLtMatmul(g_handle, p.op, &alpha, w, p.a, a, p.b, &beta, out, p.c, out, p.c, &p.algo,
                          workspace, ws, (cudaStream_t)stream));
  return ERB_OK;
}

#if ERB_ELEM == 1
// ---------------------------------------------------------------------------------------------
// Weight-streaming product for few rows (decode): out[M, N] = a[M, K] * w[N, K]^T, M <= 64,
// bfloat16 operands, float accumulation.  The work is reading w once at memory speed, so w is the
// "A" operand of mma.sync.m16n8k16 (16 rows of w per tile) and the few rows of `a` are the 8-wide
// "B" operand: no shared-memory staging, every operand fragment is a plain 16-byte global load.
//
// Fragment trick: a dot product does not care in which order k is visited, as long as both
// operands agree.  Lane (r = lane / 4, j = lane % 4) loads 8 consecutive k of w row r and of row
// r + 8, and the same 8 k of `a` row r; elements 0..3 feed one mma (as the k = 2j, 2j+1, 2j+8,
// 2j+9 slots of the instruction), elements 4..7 the next.  One pass covers 32 k with two mma.
//
// The warps of a block take passes round-robin (so together they read contiguous bytes of each row
// per round) and their partial sums are added in warp order through shared memory.
//
// An output element's bits do not depend on how many rows `a` has: the number of warps (which k a
// warp sums) is a function of N and K alone, rows of `a` beyond the first 8 only add tiles beside
// the first one, and a block that takes two tiles of w rows (for 17 rows and more, where the
// fragments of `a` are then used twice) sums each exactly as a block with one would.
// ---------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MODE 0: bfloat16 out; 1: float out; 2: gated (see erb_linear_skinny_glu): w holds N gate rows and
// then N up rows, a tile takes 8 gate rows as the first half of its 16 and the 8 up rows that go
// with them as the second, so that after the reduction one thread holds g and u of an output and
// writes silu(g) * u (both rounded to bfloat16 first, as if the product had been stored).
// MODE 3 (see erb_linear_skinny_rope): w is [Wq; Wk; Wv]; a tile of a q or k head takes 8 rows of
// the head's first half and the 8 rows half a head further on, so that one thread holds both
// elements of a rotary pair; it rotates them by the token's angle and writes q to `out` and k to
// the token's cache slot.  Tiles of v heads take 16 neighbouring rows and write them to the slot.
struct RopeArgs {
  const int* positions;        // per row of `a`
  const float* inv_freq;       // [head_dim / 2]
  const int* slots;            // per row of `a`: page * page_size + offset, negative: write no k, v
  __nv_bfloat16* k_pages;      // [page][kv head][offset][head_dim]
  __nv_bfloat16* v_pages;
  int nq, nkv, head_dim, page_size;
};

// NT: tiles of 8 rows of `a`; RT: tiles of 16 rows of w per block; kSkWarps: warps per block;
// CL: blocks that share a tile of w rows (a cluster of 1 or 2: with 2, each streams every other
// group of passes, and the second hands its sums to the first through distributed shared memory).
template <int NT, int RT, int MODE, int kSkWarps, int CL>
__global__ void __launch_bounds__(kSkWarps * 32, (NT * RT <= 2) ? 32 / kSkWarps : 1)
linear_skinny_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, void* __restrict__ out,
                     int M, int N, int K, int lda, int ldw, int ldo, int n_tiles, RopeArgs ra) {
  constexpr bool OUT_F32 = MODE == 1;
  constexpr bool GLU = MODE == 2;
  constexpr bool ROPE = MODE == 3;
  constexpr bool PAIRED = GLU || ROPE;                // a thread finishes two values (gate and up, a rotary pair) together
  constexpr int kUnroll = (NT * RT <= 2) ? 4 : 2;     // passes in flight per warp
  constexpr int kAllWarps = kSkWarps * CL;            // warps that share the k of a tile
  constexpr int kFinishers = PAIRED ? 64 : 128;       // threads that add the warps' sums: one per value (or pair)
  __shared__ float red[kSkWarps][32][4];
  __shared__ float handed[CL > 1 ? NT * RT : 1][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;
  const int rank = CL > 1 ? (int)(blockIdx.x % CL) : 0;        // (clusters are consecutive blocks)
  const int first_tile = (int)(blockIdx.x / CL) * RT;
  const int vwarp = rank * kSkWarps + warp;                    // this warp among all that share the tile's k
  const int per_head = ROPE ? ra.head_dim / 16 : 1;            // tiles per head
  const int rot_tiles = ROPE ? (ra.nq + ra.nkv) * per_head : 0;
  const uint4* w_lo[RT];
  const uint4* w_hi[RT];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) {
    const int tile = min(first_tile + rt, n_tiles - 1);   // (a block's second tile may not exist: it repeats the last)
    const int n0 = tile * (GLU ? 8 : 16);
    int row_lo = min(n0 + r, N - 1), row_hi = GLU ? N + min(n0 + r, N - 1) : min(n0 + r + 8, N - 1);
    if (ROPE && tile < rot_tiles) {
      row_lo = (tile / per_head) * ra.head_dim + (tile % per_head) * 8 + r;
      row_hi = row_lo + ra.head_dim / 2;
    }
    w_lo[rt] = reinterpret_cast<const uint4*>(w + (size_t)row_lo * ldw);
    w_hi[rt] = reinterpret_cast<const uint4*>(w + (size_t)row_hi * ldw);
  }
  const int chunks = K >> 3;                          // 16-byte chunks per row
  const int passes = (chunks + 3) >> 2;               // 4 chunks (32 k) per pass
  const uint4 zero = make_uint4(0, 0, 0, 0);
  float acc[NT][RT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][rt][i] = 0.f;

  constexpr int kStride = kAllWarps * kUnroll;
  // The weights are constants, so the first round of fragments does not depend on the kernel before
  // this one and is loaded before chain_wait(), while that kernel (a norm, an activation, the combine
  // of attention) may still be running.
  uint4 lo[kUnroll][RT], hi[kUnroll][RT];
  auto load_w = [&](int p0) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int c = (p0 + u * kAllWarps) * 4 + j;
      const bool in = c < chunks;
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        lo[u][rt] = in ? __ldcs(w_lo[rt] + c) : zero;
        hi[u][rt] = in ? __ldcs(w_hi[rt] + c) : zero;
      }
    }
  };
  load_w(vwarp);
  chain_wait();

  const uint4* a_row[NT];
  bool a_ok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    a_ok[t] = t * 8 + r < M;
    a_row[t] = reinterpret_cast<const uint4*>(a + (size_t)(a_ok[t] ? t * 8 + r : 0) * lda);
  }
  auto multiply = [&](int p0) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int c = (p0 + u * kAllWarps) * 4 + j;
      const bool in = c < chunks;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 x = (in && a_ok[t]) ? __ldg(a_row[t] + c) : zero;
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          const uint32_t a0[4] = {lo[u][rt].x, hi[u][rt].x, lo[u][rt].y, hi[u][rt].y};
          const uint32_t a1[4] = {lo[u][rt].z, hi[u][rt].z, lo[u][rt].w, hi[u][rt].w};
          mma_16816(acc[t][rt], a0, x.x, x.y);
          mma_16816(acc[t][rt], a1, x.z, x.w);
        }
      }
    }
  };
  if (vwarp < passes) multiply(vwarp);
  for (int p0 = vwarp + kStride; p0 < passes; p0 += kStride) {
    load_w(p0);
    multiply(p0);
  }

  // What becomes of a finished value (or pair of values) of tile `tile` of w and tile t of a.
  // Accumulator layout: values 0, 1 belong to w row r, values 2, 3 to row r + 8; `a` rows 2j, 2j + 1.
  auto finish = [&](int tile, int t, int idx, float v0, float v1) {
    const int n0 = tile * (GLU ? 8 : 16);
    if constexpr (PAIRED) {
      const int l = idx / 2, i = idx % 2;
      const int rr = l >> 2;
      const int m = t * 8 + (l & 3) * 2 + i;
      if (m >= M) return;
      v0 = __bfloat162float(__float2bfloat16_rn(v0));       // the product as it would have been stored
      v1 = __bfloat162float(__float2bfloat16_rn(v1));
      if constexpr (GLU) {
        const int n = n0 + rr;
        if (n < N) reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(silu_mul(v0, v1));
      } else {
        const int D = ra.head_dim, half = D / 2;
        const int slot = ra.slots[m];
        const size_t page = slot >= 0 ? slot / ra.page_size : 0, off = slot >= 0 ? slot % ra.page_size : 0;
        if (tile < rot_tiles) {
          const int head = tile / per_head, e = (tile % per_head) * 8 + rr;
          float sn, cs, o0, o1;
          sincosf((float)ra.positions[m] * ra.inv_freq[e], &sn, &cs);
          rotate_pair(v0, v1, cs, sn, o0, o1);
          __nv_bfloat16* dst = nullptr;
          if (head < ra.nq) dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + (size_t)head * D;
          else if (slot >= 0) dst = ra.k_pages + ((page * ra.nkv + (head - ra.nq)) * ra.page_size + off) * D;
          if (dst) { dst[e] = __float2bfloat16_rn(o0); dst[e + half] = __float2bfloat16_rn(o1); }
        } else if (slot >= 0) {
          const int v_el = (tile - rot_tiles) * 16 + rr;                // element of the token's v row
          __nv_bfloat16* dst = ra.v_pages + ((page * ra.nkv + v_el / D) * ra.page_size + off) * D + v_el % D;
          dst[0] = __float2bfloat16_rn(v0);
          dst[8] = __float2bfloat16_rn(v1);
        }
      }
    } else {
      const int l = idx / 4, i = idx % 4;
      const int n = n0 + (l >> 2) + ((i >> 1) << 3);
      const int m = t * 8 + (l & 3) * 2 + (i & 1);
      if (n < N && m < M) {
        if (OUT_F32) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v0;
        else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v0);
      }
    }
  };

  // The partial sums of a block's warps are added in warp order, one (tile of w, tile of a) at a time.
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) {
    const int tile = first_tile + rt;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const bool live = tile < n_tiles && t * 8 < M;       // (the same for the whole cluster)
      if (CL == 1 && !live) continue;
      if (rt + t > 0) __syncthreads();                   // (the sums of the round before have been read)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][lane][i] = acc[t][rt][i];
      __syncthreads();
      const int idx = threadIdx.x;
      if (idx < kFinishers && live) {
        float v0 = 0.f, v1 = 0.f;
        // (32 warps: the sums of the first and of the second 16 are added last, as two blocks of a cluster would)
        constexpr int kHalf = kSkWarps == 32 ? 16 : kSkWarps;
        float u0 = 0.f, u1 = 0.f;
        if constexpr (PAIRED) {
          const int l = idx / 2, i = idx % 2;
#pragma unroll
          for (int wv = 0; wv < kHalf; ++wv) { v0 += red[wv][l][i]; v1 += red[wv][l][i + 2]; }
#pragma unroll
          for (int wv = kHalf; wv < kSkWarps; ++wv) { u0 += red[wv][l][i]; u1 += red[wv][l][i + 2]; }
        } else {
          const int l = idx / 4, i = idx % 4;
#pragma unroll
          for (int wv = 0; wv < kHalf; ++wv) v0 += red[wv][l][i];
#pragma unroll
          for (int wv = kHalf; wv < kSkWarps; ++wv) u0 += red[wv][l][i];
        }
        if constexpr (kSkWarps == 32) { v0 += u0; v1 += u1; }
        if constexpr (CL == 1) {
          finish(tile, t, idx, v0, v1);
        } else {
          handed[rt * NT + t][idx] = v0;
          if (PAIRED) handed[rt * NT + t][64 + idx] = v1;
        }
      }
    }
  }
  if constexpr (CL > 1) {
    // The first block of the cluster adds the other's sums to its own (always in this order) and finishes.
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0 && threadIdx.x < kFinishers) {
      const int idx = threadIdx.x;
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(&handed[0][0])), "r"(1));
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        const int tile = first_tile + rt;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (!(tile < n_tiles && t * 8 < M)) continue;
          float o0, o1 = 0.f;
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(o0) : "r"(remote + 4u * (uint32_t)((rt * NT + t) * 128 + idx)));
          if (PAIRED) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(o1) : "r"(remote + 4u * (uint32_t)((rt * NT + t) * 128 + 64 + idx)));
          finish(tile, t, idx, handed[rt * NT + t][idx] + o0, PAIRED ? handed[rt * NT + t][64 + idx] + o1 : 0.f);
        }
      }
    }
    // the second block's shared memory must stay until the first has read it
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
}

// A launch with programmatic stream serialization and, for cluster > 1, a cluster of that many blocks.
template <typename... KArgs, typename... Args>
void launch_skinny(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (chain_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in check_launch()
}

template <int NT, int RT, int MODE>
int launch_skinny_tiles(const __nv_bfloat16* ap, const __nv_bfloat16* wp, void* out, int M, int N, int K, int lda,
                        int ldw, int ldo, cudaStream_t s, RopeArgs ra) {
  // Warps that share the k of a tile of w rows: 8; 16, or 32 (two blocks of 16 on two SMs, for rows of
  // 4096 k and more) when the product has so few rows of w that 8-warp blocks would leave the SMs short of
  // loads in flight.  A function of N and K only: their number decides which k a warp sums, and a result
  // must not depend on the number of rows of a.
  const int n_tiles = MODE == 2 ? (N + 7) / 8 : (N + 15) / 16;
  const unsigned blocks = (unsigned)((n_tiles + RT - 1) / RT);
  const unsigned sms = (unsigned)sm_count();
  if ((unsigned)n_tiles <= sms && K >= 4096) {
    // 32 warps: one block where its registers allow (up to 16 rows of a), else two blocks of 16 on two SMs
    if constexpr (NT * RT <= 2)
      launch_skinny(linear_skinny_kernel<NT, RT, MODE, 32, 1>, dim3(blocks), dim3(1024), 0, 1, s, ap, wp, out, M, N, K, lda, ldw, ldo, n_tiles, ra);
    else
      launch_skinny(linear_skinny_kernel<NT, RT, MODE, 16, 2>, dim3(2 * blocks), dim3(512), 0, 2, s, ap, wp, out, M, N, K, lda, ldw, ldo, n_tiles, ra);
  }
  else if ((unsigned)n_tiles < 2 * sms && K >= 1024)
    launch_skinny(linear_skinny_kernel<NT, RT, MODE, 16, 1>, dim3(blocks), dim3(512), 0, 1, s, ap, wp, out, M, N, K, lda, ldw, ldo, n_tiles, ra);
  else
    launch_skinny(linear_skinny_kernel<NT, RT, MODE, 8, 1>, dim3(blocks), dim3(256), 0, 1, s, ap, wp, out, M, N, K, lda, ldw, ldo, n_tiles, ra);
  return check_launch("linear_skinny");
}

// Up to 16 rows of a: a block takes one tile of w rows.  From 17 rows on (where the library or the
// tensor-core kernel is the better choice, and this kernel only keeps its contract) a block takes two
// tiles of w rows and uses every fragment of a twice.
template <int MODE>
int launch_skinny_mode(const __nv_bfloat16* ap, const __nv_bfloat16* wp, void* out, int M, int N, int K, int lda,
                       int ldw, int ldo, cudaStream_t s, RopeArgs ra = RopeArgs{}) {
  if (M <= 8) return launch_skinny_tiles<1, 1, MODE>(ap, wp, out, M, N, K, lda, ldw, ldo, s, ra);
  if (M <= 16) return launch_skinny_tiles<2, 1, MODE>(ap, wp, out, M, N, K, lda, ldw, ldo, s, ra);
  if (M <= 32) return launch_skinny_tiles<4, 2, MODE>(ap, wp, out, M, N, K, lda, ldw, ldo, s, ra);
  return launch_skinny_tiles<8, 2, MODE>(ap, wp, out, M, N, K, lda, ldw, ldo, s, ra);
}

int check_skinny(const char* who, const void* a, const void* w, int M, int N, int K, int lda, int ldw, int ldo) {
  if (M > 64) return fail(ERB_ERR_UNSUPPORTED, "%s: %d rows (at most 64)", who, M);
  if (N <= 0 || K <= 0 || lda < K || ldw < K || ldo < N) return fail(ERB_ERR_ARG, "%s: bad sizes", who);
  if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return fail(ERB_ERR_UNSUPPORTED, "%s: K and the leading dimensions must be multiples of 8", who);
  return ERB_OK;
}

}  // namespace

// Same result contract as erb_linear (no accumulate), for 1 <= M <= 64 with K, lda and ldw
// multiples of 8 elements and 16-byte aligned operands.
ERB_EXPORT int erb_linear_skinny(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw,
                                 int ldo, int out_f32, void* stream) {
  if (M <= 0) return ERB_OK;
  int rc = check_skinny("linear_skinny", a, w, M, N, K, lda, ldw, ldo);
  if (rc) return rc;
  const __nv_bfloat16 *ap = (const __nv_bfloat16*)a, *wp = (const __nv_bfloat16*)w;
  if (out_f32) return launch_skinny_mode<1>(ap, wp, out, M, N, K, lda, ldw, ldo, (cudaStream_t)stream);
  return launch_skinny_mode<0>(ap, wp, out, M, N, K, lda, ldw, ldo, (cudaStream_t)stream);
}

// The attention input projection of a decode step with the rotary encoding and the cache write in
// its epilogue: w = [Wq; Wk; Wv] of shape [(nq + 2 nkv) * head_dim, K]; q is rotated and written to
// out[M, >= nq * head_dim] (the k and v columns of `out` are not written), k is rotated and, with v,
// written to each token's cache slot.  The products are rounded to bfloat16 before the rotation, so
// the result equals erb_linear_skinny followed by the rotation kernel.  Full rotation only
// (rot_dim == head_dim), head_dim a multiple of 16, 1 <= M <= 64.
ERB_EXPORT int erb_linear_skinny_rope(const void* a, const void* w, void* out, int M, int K, int lda, int ldw, int ldo,
                                      int nq, int nkv, int head_dim, const int* positions, const float* inv_freq,
                                      const int* slots, void* k_pages, void* v_pages, int page_size, void* stream) {
  if (M <= 0) return ERB_OK;
  if (nq <= 0 || nkv <= 0 || head_dim <= 0 || head_dim % 16)
    return fail(ERB_ERR_UNSUPPORTED, "linear_skinny_rope: head_dim %d must be a multiple of 16", head_dim);
  const int N = (nq + 2 * nkv) * head_dim;
  if (page_size <= 0 || !positions || !inv_freq || !slots || !k_pages || !v_pages)
    return fail(ERB_ERR_ARG, "linear_skinny_rope: bad arguments");
  int rc = check_skinny("linear_skinny_rope", a, w, M, nq * head_dim, K, lda, ldw, ldo);
  if (rc) return rc;
  const RopeArgs ra{positions, inv_freq, slots, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, nq, nkv, head_dim, page_size};
  return launch_skinny_mode<3>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, M, N, K, lda, ldw, ldo,
                               (cudaStream_t)stream, ra);
}

// Gated product for the feed-forward of a decode step: w holds N gate rows and then N up rows
// ([2N, K]); out[M, N] = silu(g) * u with g = a * gate^T and u = a * up^T, each rounded to bfloat16
// before the gate (so the result equals erb_linear_skinny into a [M, 2N] buffer followed by the
// gate kernel), 1 <= M <= 64.
ERB_EXPORT int erb_linear_skinny_glu(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw,
                                     int ldo, void* stream) {
  if (M <= 0) return ERB_OK;
  int rc = check_skinny("linear_skinny_glu", a, w, M, N, K, lda, ldw, ldo);
  if (rc) return rc;
  return launch_skinny_mode<2>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, out, M, N, K, lda, ldw, ldo,
                               (cudaStream_t)stream);
}
#endif  // ERB_ELEM == 1
