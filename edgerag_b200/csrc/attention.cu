// Causal grouped-query attention over cache pages, for any element type and head size.
//
// These are the general kernels: CUDA-core arithmetic in float, any head size that is a multiple
// of 16 up to 256, any page size, any number of heads and groups, an optional window.  They serve
// the 32-bit path and every shape the tensor-core kernels do not take.
//
// Cache layout (one layer): pages[page][kv head][offset][D]; a token at logical position p of a
// sequence lives in page block_table[seq][p / page_size] at offset p % page_size.  Keys are
// stored already rotated.  A query at position p sees keys max(0, p - window + 1) .. p
// (window <= 0: all keys 0 .. p).  Query head h reads kv head h / (nq / nkv).
//
// Both kernels give every thread its own keys and its own online-softmax state (running max,
// denominator, float accumulator of D values), so the inner loop has no cross-thread traffic;
// states are merged once at the end, in a fixed order.
#include <mutex>

#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

template <typename T> struct Vec;  // 16-byte vectors
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* p, float* out);
template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float* out) { load4(p, out); }
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* p, float* out) { load8(p, out); }

// One thread's online-softmax state over the keys it visits.
template <int D>
struct LaneState {
  float m = -INFINITY, l = 0.f;
  float acc[D];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
  }
  // Visit one key: k and v point at the D elements of the key and the value row.
  template <typename T>
  __device__ __forceinline__ void visit(const float* q_smem, const T* k, const T* v, float scale) {
    constexpr int N = Vec<T>::N;
    float s = 0.f;
#pragma unroll
    for (int d0 = 0; d0 < D; d0 += N) {
      float kk[N];
      load_vec<T, N>(k + d0, kk);
#pragma unroll
      for (int i = 0; i < N; ++i) s = fmaf(q_smem[d0 + i], kk[i], s);
    }
    s *= scale;
    float p;
    if (s > m) {
      const float alpha = expf(m - s);  // exp(-inf) = 0 on the first key
      l *= alpha;
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] *= alpha;
      m = s;
      p = 1.f;
    } else {
      p = expf(s - m);
    }
    l += p;
#pragma unroll
    for (int d0 = 0; d0 < D; d0 += N) {
      float vv[N];
      load_vec<T, N>(v + d0, vv);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[d0 + i] = fmaf(p, vv[i], acc[d0 + i]);
    }
  }
};

// Merge the 32 states of a warp.  `stage` is the warp's shared area of 32 * (D + 1) floats.
// Afterwards lane x holds, for each i with d = x + 32 i < D, the warp's sum for column d in
// out[i]; the warp's max and denominator are returned in m_w / l_w (same on every lane).
template <int D>
__device__ __forceinline__ void warp_merge(LaneState<D>& st, float* stage, float& m_w, float& l_w,
                                           float* out /* (D + 31) / 32 */) {
  const int lane = threadIdx.x & 31;
  m_w = warp_max(st.m);
  const float f = (st.m == -INFINITY) ? 0.f : expf(st.m - m_w);
  l_w = warp_sum(st.l * f);
  float* mine = stage + lane * (D + 1);
#pragma unroll
  for (int d = 0; d < D; ++d) mine[d] = st.acc[d] * f;
  __syncwarp();
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    float sum = 0.f;
    if (d < D) {
#pragma unroll 8
      for (int j = 0; j < 32; ++j) sum += stage[j * (D + 1) + d];
    }
    out[i] = sum;
  }
  __syncwarp();
}

constexpr int kRowWarps = 4;  // warps (query rows) per block in the row kernel

// ---------------------------------------------------------------------------------------------
// Row kernel: one warp per (query token, query head).  Handles portions of prompts and decoded
// tokens alike; the only per-token inputs are its sequence and its position.
// ---------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kRowWarps * 32)
attention_rows_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_pages,
                      const T* __restrict__ v_pages, const int* __restrict__ block_tables, int max_pages,
                      const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                      T* __restrict__ out, int out_row_stride, int n_tokens, int nq, int nkv,
                      int page_size, int window, float scale) {
  chain_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * D;
  float* stage = smem + kRowWarps * D + warp * 32 * (D + 1);
  const int t = blockIdx.x * kRowWarps + warp;
  const int h = blockIdx.y;
  if (t >= n_tokens) return;  // warps are independent: no block-wide barrier below
  const T* q_row = q + (size_t)t * q_row_stride + (size_t)h * D;
  for (int d = lane; d < D; d += 32) q_s[d] = Elem<T>::load(q_row + d);
  __syncwarp();

  const int seq = seq_of_token[t], pos = positions[t];
  const int kvh = h / (nq / nkv);
  const int* bt = block_tables + (size_t)seq * max_pages;
  const int k_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  LaneState<D> st;
  st.init();
  for (int k = k_lo + lane; k <= pos; k += 32) {
    const int page = bt[k / page_size];
    const size_t row = (((size_t)page * nkv + kvh) * page_size + (k % page_size)) * D;
    st.template visit<T>(q_s, k_pages + row, v_pages + row, scale);
  }
  float m_w, l_w, o[(D + 31) / 32];
  warp_merge<D>(st, stage, m_w, l_w, o);
  const float inv = 1.f / l_w;
  T* o_row = out + (size_t)t * out_row_stride + (size_t)h * D;
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) Elem<T>::store(o_row + d, o[i] * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// Decode kernel: one query token per sequence; the keys of a sequence are cut into splits of
// `split_keys` keys, one block per (split, query head, sequence).  Partial results (max,
// denominator, unnormalised accumulator) go to scratch; the combine kernel merges the splits in
// order.  The split size is a constant of the launch, so a sequence's result does not depend on
// what else is in the batch.
// ---------------------------------------------------------------------------------------------
constexpr int kDecodeWarps = 4;

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeWarps * 32)
attention_decode_split_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ k_pages,
                              const T* __restrict__ v_pages, const int* __restrict__ block_tables,
                              int max_pages, const int* __restrict__ token_of_seq,
                              const int* __restrict__ positions, float* __restrict__ part_acc,
                              float* __restrict__ part_ml, int max_splits, int nq, int nkv, int page_size,
                              int window, int split_keys, float scale) {
  chain_wait();
  extern __shared__ float smem[];
  float* q_s = smem;                                   // D
  float* stage = smem + D;                             // kDecodeWarps * 32 * (D + 1)
  float* warp_out = stage + kDecodeWarps * 32 * (D + 1);  // kDecodeWarps * (D + 2)
  const int split = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = token_of_seq[seq];
  const int pos = positions[t];
  const int k_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // Splits are aligned to multiples of split_keys in absolute key positions.
  const int first_split = k_lo / split_keys;
  const int begin = max(k_lo, (first_split + split) * split_keys);
  const int end = min(pos + 1, (first_split + split + 1) * split_keys);
  if (begin >= end) return;  // this split does not exist for this sequence

  const T* q_row = q + (size_t)t * q_row_stride + (size_t)h * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) q_s[d] = Elem<T>::load(q_row + d);
  __syncthreads();

  const int kvh = h / (nq / nkv);
  const int* bt = block_tables + (size_t)seq * max_pages;
  LaneState<D> st;
  st.init();
  for (int k = begin + (int)threadIdx.x; k < end; k += kDecodeWarps * 32) {
    const int page = bt[k / page_size];
    const size_t row = (((size_t)page * nkv + kvh) * page_size + (k % page_size)) * D;
    st.template visit<T>(q_s, k_pages + row, v_pages + row, scale);
  }
  float m_w, l_w, o[(D + 31) / 32];
  warp_merge<D>(st, stage + warp * 32 * (D + 1), m_w, l_w, o);
  float* wo = warp_out + warp * (D + 2);
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) wo[d] = o[i];
  }
  if (lane == 0) { wo[D] = m_w; wo[D + 1] = l_w; }
  __syncthreads();
  // Merge the warps in order.
  float m_b = -INFINITY;
#pragma unroll
  for (int w = 0; w < kDecodeWarps; ++w) m_b = fmaxf(m_b, warp_out[w * (D + 2) + D]);
  const size_t slot = ((size_t)seq * nq + h) * max_splits + split;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float mw = warp_out[w * (D + 2) + D];
      const float f = (mw == -INFINITY) ? 0.f : expf(mw - m_b);
      sum += warp_out[w * (D + 2) + d] * f;
    }
    part_acc[slot * D + d] = sum;
  }
  if (threadIdx.x == 0) {
    float l_b = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float mw = warp_out[w * (D + 2) + D];
      const float f = (mw == -INFINITY) ? 0.f : expf(mw - m_b);
      l_b += warp_out[w * (D + 2) + D + 1] * f;
    }
    part_ml[slot * 2] = m_b;
    part_ml[slot * 2 + 1] = l_b;
  }
}

template <typename T>
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_acc,
                                                const float* __restrict__ part_ml,
                                                const int* __restrict__ token_of_seq,
                                                const int* __restrict__ positions, T* __restrict__ out,
                                                int out_row_stride, int max_splits, int nq, int head_dim,
                                                int window, int split_keys) {
  chain_wait();
  const int h = blockIdx.x, seq = blockIdx.y;
  const int t = token_of_seq[seq];
  const int pos = positions[t];
  const int k_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // never beyond what the split kernel's grid wrote (a caller that understates max_splits gets the
  // first max_splits splits merged, not its neighbours' scratch)
  const int n_splits = min(pos / split_keys - k_lo / split_keys + 1, max_splits);
  const size_t base = ((size_t)seq * nq + h) * max_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) l += part_ml[(base + s) * 2 + 1] * expf(part_ml[(base + s) * 2] - m);
  const float inv = 1.f / l;
  T* o_row = out + (size_t)t * out_row_stride + (size_t)h * head_dim;
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float sum = 0.f;
    for (int s = 0; s < n_splits; ++s)
      sum += part_acc[(base + s) * head_dim + d] * expf(part_ml[(base + s) * 2] - m);
    Elem<T>::store(o_row + d, sum * inv);
  }
}

template <typename T, int D>
int launch_rows(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                const int* block_tables, int max_pages, const int* seq_of_token, const int* positions,
                void* out, int out_row_stride, int n_tokens, int nq, int nkv, int page_size, int window,
                float scale, cudaStream_t s) {
  const size_t smem = (size_t)(kRowWarps * D + kRowWarps * 32 * (D + 1)) * sizeof(float);
  auto kern = attention_rows_kernel<T, D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_rows: %s", cudaGetErrorString(e));
  }
  dim3 grid((n_tokens + kRowWarps - 1) / kRowWarps, nq);
  launch_chained(kern, dim3(grid), dim3(kRowWarps * 32), smem, s, (const T*)q, q_row_stride, (const T*)k_pages, (const T*)v_pages,
      block_tables, max_pages, seq_of_token, positions, (T*)out, out_row_stride, n_tokens, nq, nkv,
      page_size, window, scale);
  return check_launch("attention_rows");
}

template <typename T, int D>
int launch_decode(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                  const int* block_tables, int max_pages, const int* token_of_seq, const int* positions,
                  void* out, int out_row_stride, float* part_acc, float* part_ml, int max_splits, int n_seqs,
                  int nq, int nkv, int page_size, int window, int split_keys, float scale, cudaStream_t s) {
  const size_t smem =
      (size_t)(D + kDecodeWarps * 32 * (D + 1) + kDecodeWarps * (D + 2)) * sizeof(float);
  auto kern = attention_decode_split_kernel<T, D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_decode: %s", cudaGetErrorString(e));
  }
  dim3 grid(max_splits, nq, n_seqs);
  launch_chained(kern, dim3(grid), dim3(kDecodeWarps * 32), smem, s, (const T*)q, q_row_stride, (const T*)k_pages,
      (const T*)v_pages, block_tables, max_pages, token_of_seq, positions, part_acc, part_ml, max_splits,
      nq, nkv, page_size, window, split_keys, scale);
  int rc = check_launch("attention_decode_split");
  if (rc) return rc;
  launch_chained(attention_decode_combine_kernel<T>, dim3(dim3(nq, n_seqs)), dim3(64), 0, s, part_acc, part_ml, token_of_seq,
      positions, (T*)out, out_row_stride, max_splits, nq, D, window, split_keys);
  return check_launch("attention_decode_combine");
}

int check_common(const char* who, int nq, int nkv, int head_dim, int page_size, int max_pages) {
  if (nq <= 0 || nkv <= 0 || nq % nkv) return fail(ERB_ERR_ARG, "%s: %d query heads / %d kv heads", who, nq, nkv);
  if (head_dim < 16 || head_dim > 256 || head_dim % 16)
    return fail(ERB_ERR_UNSUPPORTED, "%s: head_dim %d is not a multiple of 16 in [16, 256]", who, head_dim);
  if (page_size <= 0 || max_pages <= 0) return fail(ERB_ERR_ARG, "%s: bad page_size/max_pages", who);
  return ERB_OK;
}

}  // namespace

#define ERB_DISPATCH_D(FN, ...)                                                                \
  switch (head_dim) {                                                                          \
    case 16: return FN<elem_t, 16>(__VA_ARGS__);   case 32: return FN<elem_t, 32>(__VA_ARGS__);   \
    case 48: return FN<elem_t, 48>(__VA_ARGS__);   case 64: return FN<elem_t, 64>(__VA_ARGS__);   \
    case 80: return FN<elem_t, 80>(__VA_ARGS__);   case 96: return FN<elem_t, 96>(__VA_ARGS__);   \
    case 112: return FN<elem_t, 112>(__VA_ARGS__); case 128: return FN<elem_t, 128>(__VA_ARGS__); \
    case 144: return FN<elem_t, 144>(__VA_ARGS__); case 160: return FN<elem_t, 160>(__VA_ARGS__); \
    case 176: return FN<elem_t, 176>(__VA_ARGS__); case 192: return FN<elem_t, 192>(__VA_ARGS__); \
    case 208: return FN<elem_t, 208>(__VA_ARGS__); case 224: return FN<elem_t, 224>(__VA_ARGS__); \
    case 240: return FN<elem_t, 240>(__VA_ARGS__); case 256: return FN<elem_t, 256>(__VA_ARGS__); \
  }

// q: [n_tokens, ...] with `q_row_stride` elements between rows, head h at column h * head_dim.
// out: the same shape convention.  block_tables: int32 [n_seqs, max_pages].
ERB_EXPORT int erb_attention_rows(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                  const int* block_tables, int max_pages, const int* seq_of_token,
                                  const int* positions, void* out, int out_row_stride, int n_tokens, int nq,
                                  int nkv, int head_dim, int page_size, int window, float scale,
                                  void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  int rc = check_common("attention_rows", nq, nkv, head_dim, page_size, max_pages);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  ERB_DISPATCH_D(launch_rows, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, seq_of_token,
                 positions, out, out_row_stride, n_tokens, nq, nkv, page_size, window, scale, s)
  return fail(ERB_ERR_UNSUPPORTED, "attention_rows: head_dim %d", head_dim);
}

// Scratch the caller provides: part_acc float [n_seqs * nq * max_splits * head_dim],
// part_ml float [n_seqs * nq * max_splits * 2], with max_splits >= the largest number of splits
// any sequence of the batch has (its visible key range cut at multiples of split_keys).
ERB_EXPORT int erb_attention_decode(const void* q, int q_row_stride, const void* k_pages,
                                    const void* v_pages, const int* block_tables, int max_pages,
                                    const int* token_of_seq, const int* positions, void* out,
                                    int out_row_stride, float* part_acc, float* part_ml, int max_splits,
                                    int n_seqs, int nq, int nkv, int head_dim, int page_size, int window,
                                    int split_keys, float scale, void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  int rc = check_common("attention_decode", nq, nkv, head_dim, page_size, max_pages);
  if (rc) return rc;
  if (max_splits <= 0 || split_keys <= 0 || !part_acc || !part_ml)
    return fail(ERB_ERR_ARG, "attention_decode: scratch or split arguments missing");
  if (n_seqs > 65535 || nq > 65535) return fail(ERB_ERR_UNSUPPORTED, "attention_decode: grid too large");
  cudaStream_t s = (cudaStream_t)stream;
  ERB_DISPATCH_D(launch_decode, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                 positions, out, out_row_stride, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size,
                 window, split_keys, scale, s)
  return fail(ERB_ERR_UNSUPPORTED, "attention_decode: head_dim %d", head_dim);
}

// ---------------------------------------------------------------------------------------------
// The variant for callers that cannot allocate: scratch in a file-scope device array.
// See attention_noalloc.h for the contract.
// ---------------------------------------------------------------------------------------------
#include "attention_noalloc.h"

static __device__ __align__(256) float g_static_decode_scratch[ERB_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the array on each device; looked up once per device by the first call there.
// In host code the array's name is only a handle for the runtime, not a device pointer.
float* g_static_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_static: device %d", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_decode_scratch);
    if (e != cudaSuccess || !p)
      return fail(ERB_ERR_CUDA, "attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return ERB_OK;
}
}  // namespace

ERB_EXPORT long long erb_attention_decode_static_floats(int n_seqs, int nq, int head_dim, int max_splits) {
  return (long long)n_seqs * nq * max_splits * (head_dim + 2);
}

ERB_EXPORT int erb_attention_decode_static(const void* q, int q_row_stride, const void* k_pages,
                                           const void* v_pages, const int* block_tables, int max_pages,
                                           const int* token_of_seq, const int* positions, void* out,
                                           int out_row_stride, int max_splits, int n_seqs, int nq, int nkv,
                                           int head_dim, int page_size, int window, int split_keys,
                                           float scale, void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  if (max_splits <= 0 || nq <= 0 || head_dim <= 0)
    return fail(ERB_ERR_ARG, "attention_decode_static: bad sizes");
  const long long need = erb_attention_decode_static_floats(n_seqs, nq, head_dim, max_splits);
  if (need > (long long)ERB_STATIC_SCRATCH_FLOATS)
    return fail(ERB_ERR_UNSUPPORTED,
                "attention_decode_static: %lld floats of scratch needed (sequences %d x heads %d x splits %d x "
                "(head_dim %d + 2)), the built-in array holds %d; use erb_attention_decode with caller scratch",
                need, n_seqs, nq, max_splits, head_dim, (int)ERB_STATIC_SCRATCH_FLOATS);
  float* base = nullptr;
  int rc = static_scratch_for_current_device(&base);
  if (rc) return rc;
  float* part_acc = base;
  float* part_ml = base + (size_t)n_seqs * nq * max_splits * head_dim;
  return erb_attention_decode(q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                              positions, out, out_row_stride, part_acc, part_ml, max_splits, n_seqs, nq, nkv,
                              head_dim, page_size, window, split_keys, scale, stream);
}
