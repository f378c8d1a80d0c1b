// Row-wise kernels of the decoder step: embedding rows, residual add + RMSNorm, rotary position
// encoding fused with the write of keys and values into cache pages, and the SwiGLU gate.
//
// The residual stream is held in 32-bit for both element types; `T` is the type of everything
// that feeds a matrix product (bfloat16 on the serving path, float on the 32-bit path).
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

// ---------------------------------------------------------------------------------------------
// Embedding: hidden[t, :] = table[ids[t], :]  or  embeds[embed_row[t], :]   (written as float)
// An id outside [0, vocab) sets *status = 1 + t and writes zeros; nothing is read out of range.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(float* __restrict__ hidden, const T* __restrict__ table,
                                  const T* __restrict__ embeds, const int* __restrict__ ids,
                                  const int* __restrict__ embed_row, int hidden_size, int vocab,
                                  int n_embed_rows, int* __restrict__ status) {
  const int t = blockIdx.x;
  const int er = embed_row ? embed_row[t] : -1;
  const T* src = nullptr;
  if (er >= 0) {
    if (er < n_embed_rows && embeds) src = embeds + (size_t)er * hidden_size;
  } else {
    const int id = ids[t];
    if (id >= 0 && id < vocab) src = table + (size_t)id * hidden_size;
  }
  if (!src && threadIdx.x == 0) atomicCAS(status, 0, 1 + t);
  float* dst = hidden + (size_t)t * hidden_size;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) dst[i] = src ? Elem<T>::load(src + i) : 0.f;
}

ERB_EXPORT int erb_embed_rows(void* hidden, const void* table, const void* embeds, const int* ids,
                              const int* embed_row, int n_tokens, int hidden_size, int vocab,
                              int n_embed_rows, int* status, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (hidden_size <= 0 || vocab <= 0) return fail(ERB_ERR_ARG, "embed_rows: bad sizes");
  const int threads = hidden_size >= 1024 ? 256 : 128;
  embed_rows_kernel<elem_t><<<n_tokens, threads, 0, (cudaStream_t)stream>>>((float*)hidden,
      (const elem_t*)table, (const elem_t*)embeds, ids, embed_row, hidden_size, vocab, n_embed_rows, status);
  return check_launch("embed_rows");
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   r = hidden[row] (+ delta[row])            in float, stored back when `write_back`
//   y = weight * round_T( r * rsqrt(mean(r^2) + eps) )     rounded to T once more
// The statistics, the scale and the residual sum are float; the cast to T comes before the
// weight multiply, as in the reference's RMSNorm.  `rows`, when given, selects the rows of
// hidden/delta that are read (output row i comes from input row rows[i]).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden_size, float eps,
                                   int write_back) {
  extern __shared__ float row_cache[];  // hidden_size floats, then 32 of scratch
  float* scratch = row_cache + hidden_size;
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * hidden_size;
  const T* d = delta ? delta + (size_t)r * hidden_size : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = h[i];
    if (d) v += Elem<T>::load(d + i);
    row_cache[i] = v;
    if (write_back && d) h[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float rs = rsqrtf(total / (float)hidden_size + eps);
  T* y = out + (size_t)o * hidden_size;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    const float normed = Elem<T>::round(row_cache[i] * rs);
    Elem<T>::store(y + i, weight[i] * normed);
  }
}

ERB_EXPORT int erb_add_rmsnorm(void* hidden, const void* delta, const float* weight, void* out,
                               const int* rows, int n_rows, int hidden_size, float eps, int write_back,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  const size_t smem = (size_t)(hidden_size + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "add_rmsnorm: hidden_size %d too large", hidden_size);
  if (rows && write_back) return fail(ERB_ERR_ARG, "add_rmsnorm: row selection cannot write back");
  const int threads = hidden_size >= 4096 ? 512 : (hidden_size >= 512 ? 256 : 128);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<elem_t>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
  }
  add_rmsnorm_kernel<elem_t><<<n_rows, threads, smem, (cudaStream_t)stream>>>((float*)hidden,
      (const elem_t*)delta, weight, (elem_t*)out, rows, hidden_size, eps, write_back);
  return check_launch("add_rmsnorm");
}

// hidden[row] += delta[row] without a norm (the last residual of a stack that ends without one).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += Elem<T>::load(delta + i);
}

ERB_EXPORT int erb_residual_add(void* hidden, const void* delta, long long n, void* stream) {
  if (n <= 0) return ERB_OK;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  residual_add_kernel<elem_t><<<blocks, threads, 0, (cudaStream_t)stream>>>((float*)hidden,
      (const elem_t*)delta, (size_t)n);
  return check_launch("residual_add");
}

// ---------------------------------------------------------------------------------------------
// Rotary position encoding (halves convention) + cache write.
//   qkv: [n_tokens, (nq + 2 nkv) * D], rows hold q heads, then k heads, then v heads.
//   angle[j] = position * inv_freq[j] (float), j < rot_dim / 2; the pair is (x[j], x[j + rot/2]).
//   q is rotated in place.  k is rotated and, with v, written to the token's cache slot:
//   slot = page * page_size + offset (negative: the token writes nothing), page layout
//   [page][kv head][offset][D].  With `write_kv == 0` only q is rotated (the layer reads the
//   cache of another layer); with `rot_dim == 0` nothing is rotated (another position encoding
//   acted before) and the kernel is only the cache write.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                        int head_dim, int rot_dim, int page_size, int write_kv) {
  const int t = blockIdx.x;
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const float pos = (float)positions[t];
  const int half_rot = rot_dim / 2;
  const int half_all = head_dim / 2;  // work items per head: one per pair of elements
  const int slot = (write_kv && slots) ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? (int)(slot % page_size) : 0;

  const int rot_heads = nq + nkv;
  // q and k heads: pairs (j, j + half_rot) inside the rotated part, pass-through pairs beyond it.
  for (int w = threadIdx.x; w < rot_heads * half_all; w += blockDim.x) {
    const int head = w / half_all, j = w % half_all;
    T* x = row + (size_t)head * head_dim;
    int i0, i1;
    float o0, o1;
    if (j < half_rot) {
      i0 = j; i1 = j + half_rot;
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      const float a = Elem<T>::load(x + i0), b = Elem<T>::load(x + i1);
      o0 = a * cs - b * sn;
      o1 = b * cs + a * sn;
    } else {
      i0 = rot_dim + 2 * (j - half_rot); i1 = i0 + 1;
      o0 = Elem<T>::load(x + i0); o1 = Elem<T>::load(x + i1);
    }
    if (head < nq) {
      if (j < half_rot) { Elem<T>::store(x + i0, o0); Elem<T>::store(x + i1, o1); }
    } else if (slot >= 0) {
      const int kvh = head - nq;
      T* dst = k_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim;
      Elem<T>::store(dst + i0, o0);
      Elem<T>::store(dst + i1, o1);
    }
  }
  if (slot >= 0) {
    const T* v = row + (size_t)(nq + nkv) * head_dim;
    for (int w = threadIdx.x; w < nkv * head_dim; w += blockDim.x) {
      const int kvh = w / head_dim, i = w % head_dim;
      v_pages[(((size_t)page * nkv + kvh) * page_size + offset) * head_dim + i] = v[w];
    }
  }
}

ERB_EXPORT int erb_rope_cache_write(void* qkv, const int* positions, const float* inv_freq,
                                    const int* slots, void* k_pages, void* v_pages, int n_tokens,
                                    int nq, int nkv, int head_dim, int rot_dim, int page_size,
                                    int write_kv, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (head_dim <= 0 || head_dim % 2 || rot_dim < 0 || rot_dim > head_dim || rot_dim % 2)
    return fail(ERB_ERR_ARG, "rope_cache_write: head_dim %d / rot_dim %d must be even, rot <= head", head_dim, rot_dim);
  if (rot_dim > 0 && !inv_freq) return fail(ERB_ERR_ARG, "rope_cache_write: inv_freq missing");
  if (write_kv && (!slots || !k_pages || !v_pages || page_size <= 0))
    return fail(ERB_ERR_ARG, "rope_cache_write: cache arguments missing");
  const int work = (nq + nkv) * head_dim / 2;
  const int threads = work >= 512 ? 256 : 128;
  rope_cache_write_kernel<elem_t><<<n_tokens, threads, 0, (cudaStream_t)stream>>>((elem_t*)qkv, positions,
      inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, rot_dim, page_size, write_kv);
  return check_launch("rope_cache_write");
}

// ---------------------------------------------------------------------------------------------
// SwiGLU gate: out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], computed in float.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx % inter);
  const T* row = gate_up + t * 2 * (size_t)inter;
  const float g = Elem<T>::load(row + i), u = Elem<T>::load(row + inter + i);
  const float act = g / (1.f + expf(-g));
  Elem<T>::store(out + idx, act * u);
}

ERB_EXPORT int erb_swiglu(const void* gate_up, void* out, int n_tokens, int inter, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (inter <= 0) return fail(ERB_ERR_ARG, "swiglu: bad intermediate size");
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  swiglu_kernel<elem_t><<<blocks, threads, 0, (cudaStream_t)stream>>>((const elem_t*)gate_up, (elem_t*)out,
                                                                     inter, total);
  return check_launch("swiglu");
}

// Rows of a float matrix gathered and cast to T (the rows whose logits are wanted, when the
// stack ends without a norm).
template <typename T>
__global__ void gather_cast_kernel(const float* __restrict__ src, T* __restrict__ dst,
                                   const int* __restrict__ rows, int width) {
  const int o = blockIdx.x;
  const float* s = src + (size_t)(rows ? rows[o] : o) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(dst + (size_t)o * width + i, s[i]);
}

ERB_EXPORT int erb_gather_cast(const float* src, void* dst, const int* rows, int n_rows, int width,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  gather_cast_kernel<elem_t><<<n_rows, 256, 0, (cudaStream_t)stream>>>(src, (elem_t*)dst, rows, width);
  return check_launch("gather_cast");
}
