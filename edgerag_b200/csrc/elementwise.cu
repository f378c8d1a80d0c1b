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
  chain_wait();
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
  launch_chained(embed_rows_kernel<elem_t>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden,
      (const elem_t*)table, (const elem_t*)embeds, ids, embed_row, hidden_size, vocab, n_embed_rows, status);
  return check_launch("embed_rows");
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   r = hidden[row] (+ delta[row])            in float, stored back when `write_back`
// The update may also come as `n_parts` float arrays of partial sums, `part_stride` floats apart (a
// product whose k was split over blocks): delta = round_T(((p0 + p1) + p2) + ...), added in float in that
// order and rounded to T once, as if the product had been stored in T like every other update.
//   y = weight * round_T( r * rsqrt(mean(r^2) + eps) )     rounded to T once more
// The statistics, the scale and the residual sum are float; the cast to T comes before the
// weight multiply, as in the reference's RMSNorm.  `rows`, when given, selects the rows of
// hidden/delta that are read (output row i comes from input row rows[i]).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                   const float* __restrict__ parts, int n_parts, size_t part_stride,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden_size, float eps,
                                   int write_back) {
  chain_wait();
  extern __shared__ float row_cache[];  // hidden_size floats, then 32 of scratch
  float* scratch = row_cache + hidden_size;
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;
  float* h = hidden + (size_t)r * hidden_size;
  const T* d = delta ? delta + (size_t)r * hidden_size : nullptr;
  const float* ps = parts ? parts + (size_t)r * hidden_size : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = h[i];
    if (d) v += Elem<T>::load(d + i);
    if (ps) {
      float sum = ps[i];
      for (int sp = 1; sp < n_parts; ++sp) sum += ps[sp * part_stride + i];
      v += Elem<T>::round(sum);
    }
    row_cache[i] = v;
    if (write_back && (d || ps)) h[i] = v;
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

// Four elements per thread and step (hidden_size a multiple of 4): 16-byte accesses to the residual.
template <typename T> struct Pack4;
template <> struct Pack4<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Pack4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
};

// The same with 16-byte accesses.  The order in which a row's squares are added is that of VT
// "virtual threads" (element group g of the row belongs to virtual thread g % VT; warp trees over
// 32 neighbouring virtual threads, then one tree over the warp sums), whatever the number of real
// threads: a block of VT / R threads keeps R partial sums per thread, one per virtual thread it
// stands for.  So the launch may use fewer, busier threads for many rows and more threads for the
// few rows of a decode step, and a row's result does not depend on which.
// REGS: the row fits one pass (hidden_size <= 4 * VT), so a thread keeps its elements in registers between
// the sum and the scaling instead of parking the row in shared memory; the sums are the same.
// PARTS: the update is the sum of partial sums (see above) instead of `delta`.
template <typename T, int R, bool REGS, bool PARTS = false>
__global__ void __launch_bounds__(512, ((REGS && R > 1) || PARTS) ? 2 : 4)   // (32 registers where 2,048 threads stay resident)
add_rmsnorm_vec4_kernel(float* __restrict__ hidden, const T* __restrict__ delta,
                                        const float* __restrict__ parts, int n_parts, size_t part_stride,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        const int* __restrict__ rows, int hidden_size, float eps,
                                        int write_back, int settled) {
  extern __shared__ float row_cache[];
  float* scratch = REGS ? row_cache : row_cache + hidden_size;
  float keep[REGS ? R : 1][4];
  const int o = blockIdx.x;
  const int r = rows ? rows[o] : o;            // the step's metadata: not written by the kernel before
  float* h = hidden + (size_t)r * hidden_size;
  const T* d = (!PARTS && delta) ? delta + (size_t)r * hidden_size : nullptr;
  const float* ps = PARTS ? parts + (size_t)r * hidden_size : nullptr;
  const int threads = blockDim.x, vt = threads * R;
  // the norm's weight is a constant: this thread's first four are loaded before the wait
  const int i_first = threadIdx.x * 4;
  float w_first[4] = {0.f, 0.f, 0.f, 0.f};
  if (i_first < hidden_size) load4(weight + i_first, w_first);
  // `settled`: the residual stream was last written two or more kernels ago (the kernel just before this
  // one wrote `delta` only), so its rows may be read while that kernel is still running.
  if constexpr (REGS) {
    if (settled) {
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int i = (threadIdx.x + q * threads) * 4;
        if (i < hidden_size) load4(h + i, keep[q]);
      }
    }
  }
  chain_wait();
  float ss[R];
#pragma unroll
  for (int q = 0; q < R; ++q) ss[q] = 0.f;
  for (int base = 0; base < hidden_size; base += vt * 4) {
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int i = base + (threadIdx.x + q * threads) * 4;
      if (i >= hidden_size) continue;
      float v[4];
      if (REGS && settled) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = keep[q][j];
      } else {
        load4(h + i, v);
      }
      if constexpr (PARTS) {
        float dv[4];
        load4(ps + i, dv);
#pragma unroll 4
        for (int sp = 1; sp < n_parts; ++sp) {
          float pv[4];
          load4(ps + sp * part_stride + i, pv);
#pragma unroll
          for (int j = 0; j < 4; ++j) dv[j] += pv[j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += Elem<T>::round(dv[j]);
        if (write_back) *reinterpret_cast<float4*>(h + i) = make_float4(v[0], v[1], v[2], v[3]);
      } else if (d) {
        float dv[4];
        Pack4<T>::load(d + i, dv);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += dv[j];
        if (write_back) *reinterpret_cast<float4*>(h + i) = make_float4(v[0], v[1], v[2], v[3]);
      }
      if constexpr (REGS) {
#pragma unroll
        for (int j = 0; j < 4; ++j) keep[q][j] = v[j];
      } else {
        *reinterpret_cast<float4*>(row_cache + i) = make_float4(v[0], v[1], v[2], v[3]);
      }
      ss[q] += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
  }
  // block_sum over the virtual threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = threads >> 5;
#pragma unroll
  for (int q = 0; q < R; ++q) ss[q] = warp_sum(ss[q]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int q = 0; q < R; ++q) scratch[warp + q * warps] = ss[q];
  }
  __syncthreads();
  const float total = warp_sum(lane < warps * R ? scratch[lane] : 0.f);
  const float rs = rsqrtf(total / (float)hidden_size + eps);
  T* y = out + (size_t)o * hidden_size;
  if constexpr (REGS) {
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int i = (threadIdx.x + q * threads) * 4;
      if (i >= hidden_size) continue;
      float w[4], v[4];
      if (q == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = w_first[j];
      } else {
        load4(weight + i, w);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = w[j] * Elem<T>::round(keep[q][j] * rs);
      Pack4<T>::store(y + i, v);
    }
    return;
  }
  for (int i = threadIdx.x * 4; i < hidden_size; i += threads * 4) {
    float v[4], w[4];
    load4(row_cache + i, v);
    if (i == i_first) {
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = w_first[j];
    } else {
      load4(weight + i, w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = w[j] * Elem<T>::round(v[j] * rs);
    Pack4<T>::store(y + i, v);
  }
}

namespace {
int run_add_rmsnorm(void* hidden, const void* delta, const float* parts, int n_parts, size_t part_stride,
                    const float* weight, void* out, const int* rows, int n_rows, int hidden_size, float eps,
                    int write_back, int settled, void* stream) {
  if (n_rows <= 0) return ERB_OK;
  const size_t smem = (size_t)(hidden_size + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "add_rmsnorm: hidden_size %d too large", hidden_size);
  if (rows && write_back) return fail(ERB_ERR_ARG, "add_rmsnorm: row selection cannot write back");
  // The order of a row's sum depends on the width only (this many virtual threads), whatever the batch;
  // at 2048 and more, one pass of 16-byte loads per thread (the row's latency is paid once).
  const int threads = hidden_size >= 2048 ? 512 : (hidden_size >= 512 ? 256 : 128);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<elem_t>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
  }
  const bool vec = hidden_size % 4 == 0 && !((uintptr_t)hidden & 15) && !((uintptr_t)delta & 7) &&
                   !((uintptr_t)out & 7) && !((uintptr_t)weight & 15) && !((uintptr_t)parts & 15) && part_stride % 4 == 0;
  if (vec && parts) {
    const bool one_pass = hidden_size <= threads * 4;
    const size_t small = 32 * sizeof(float);
    if (one_pass) {
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, true, true>, dim3(n_rows), dim3(threads), small, (cudaStream_t)stream,
          (float*)hidden, (const elem_t*)nullptr, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps,
          write_back, settled);
    } else {
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 1, false, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
      }
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, false, true>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream,
          (float*)hidden, (const elem_t*)nullptr, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps,
          write_back, settled);
    }
  } else if (vec) {
    // many rows of 2048 and more: half the threads, two virtual threads each (same sums, see the kernel)
    const bool halve = threads == 512 && n_rows > 64;
    const bool one_pass = hidden_size <= threads * 4;     // a row fits the registers of its block
    if (smem > 48 * 1024 && !one_pass) {
      cudaError_t e = halve ? cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(add_rmsnorm_vec4_kernel<elem_t, 1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "add_rmsnorm: %s", cudaGetErrorString(e));
    }
    const size_t small = 32 * sizeof(float);
    if (halve && one_pass)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 2, true>, dim3(n_rows), dim3(256), small, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled);
    else if (halve)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 2, false>, dim3(n_rows), dim3(256), smem, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled);
    else if (one_pass)
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, true>, dim3(n_rows), dim3(threads), small, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled);
    else
      launch_chained(add_rmsnorm_vec4_kernel<elem_t, 1, false>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream, (float*)hidden,
          (const elem_t*)delta, nullptr, 0, (size_t)0, weight, (elem_t*)out, rows, hidden_size, eps, write_back, settled);
  } else {
    launch_chained(add_rmsnorm_kernel<elem_t>, dim3(n_rows), dim3(threads), smem, (cudaStream_t)stream, (float*)hidden,
        (const elem_t*)delta, parts, n_parts, part_stride, weight, (elem_t*)out, rows, hidden_size, eps, write_back);
  }
  return check_launch("add_rmsnorm");
}
}  // namespace

ERB_EXPORT int erb_add_rmsnorm(void* hidden, const void* delta, const float* weight, void* out,
                               const int* rows, int n_rows, int hidden_size, float eps, int write_back,
                               int settled, void* stream) {
  return run_add_rmsnorm(hidden, delta, nullptr, 0, 0, weight, out, rows, n_rows, hidden_size, eps, write_back, settled, stream);
}

// The same with the update given as `n_parts` arrays of partial sums [rows of hidden][hidden_size], float,
// `part_stride` floats from one to the next; they are added in their order.
ERB_EXPORT int erb_add_rmsnorm_parts(void* hidden, const float* parts, int n_parts, long long part_stride, const float* weight,
                                     void* out, const int* rows, int n_rows, int hidden_size, float eps, int write_back,
                                     int settled, void* stream) {
  if (!parts || n_parts < 1 || part_stride < 0) return fail(ERB_ERR_ARG, "add_rmsnorm_parts: bad arguments");
  return run_add_rmsnorm(hidden, nullptr, parts, n_parts, (size_t)part_stride, weight, out, rows, n_rows, hidden_size, eps,
                         write_back, settled, stream);
}

// hidden[row] += delta[row] without a norm (the last residual of a stack that ends without one).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ hidden, const T* __restrict__ delta, size_t n) {
  chain_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) hidden[i] += Elem<T>::load(delta + i);
}

// hidden += round_T(p0 + p1 + ...) for float partial sums, `part_stride` floats apart.
template <typename T>
__global__ void residual_add_parts_kernel(float* __restrict__ hidden, const float* __restrict__ parts, int n_parts,
                                          size_t part_stride, size_t n) {
  chain_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float sum = parts[i];
  for (int sp = 1; sp < n_parts; ++sp) sum += parts[sp * part_stride + i];
  hidden[i] += Elem<T>::round(sum);
}

ERB_EXPORT int erb_residual_add_parts(void* hidden, const float* parts, int n_parts, long long part_stride, long long n,
                                      void* stream) {
  if (n <= 0) return ERB_OK;
  if (!parts || n_parts < 1 || part_stride < 0) return fail(ERB_ERR_ARG, "residual_add_parts: bad arguments");
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  launch_chained(residual_add_parts_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden, parts,
      n_parts, (size_t)part_stride, (size_t)n);
  return check_launch("residual_add_parts");
}

ERB_EXPORT int erb_residual_add(void* hidden, const void* delta, long long n, void* stream) {
  if (n <= 0) return ERB_OK;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  launch_chained(residual_add_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (float*)hidden,
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
  chain_wait();
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
      rotate_pair(a, b, cs, sn, o0, o1);
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

// Sixteen bytes of consecutive elements as floats, and back (8 bfloat16 or 4 float).
template <typename T> struct Wide;
template <> struct Wide<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) { Pack4<float>::store(p, v); }
};
template <> struct Wide<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { load8(p, v); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// Full rotation (rot_dim == head_dim, a multiple of 2 * Wide<T>::N): the angles of a token are computed
// once per block into shared memory, every work item moves sixteen bytes of each half, and the heads of
// a token are spread over gridDim.y blocks so that a few decode tokens still fill the GPU.
template <typename T>
__global__ void rope_cache_write_wide_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                             int head_dim, int page_size, int write_kv) {
  constexpr int N = Wide<T>::N;
  extern __shared__ float trig[];            // cos[half], sin[half]
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], trig + half + j, trig + j);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  __syncthreads();
  chain_wait();
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? slot % page_size : 0;
  const int per_head = half / N;              // items per rotated head
  const int rot_items = (nq + nkv) * per_head;
  const int v_items = slot >= 0 ? nkv * head_dim / N : 0;
  const int stride = gridDim.y * blockDim.x;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < rot_items + v_items; w += stride) {
    if (w < rot_items) {
      const int head = w / per_head, j = (w % per_head) * N;
      if (head >= nq && slot < 0) continue;
      T* x = row + (size_t)head * head_dim;
      float a[N], b[N], lo[N], hi[N];
      Wide<T>::load(x + j, a);
      Wide<T>::load(x + j + half, b);
#pragma unroll
      for (int i = 0; i < N; ++i) rotate_pair(a[i], b[i], trig[j + i], trig[half + j + i], lo[i], hi[i]);
      T* dst = x;
      if (head >= nq) dst = k_pages + (((size_t)page * nkv + (head - nq)) * page_size + offset) * head_dim;
      Wide<T>::store(dst + j, lo);
      Wide<T>::store(dst + j + half, hi);
    } else {
      const int i = (w - rot_items) * N;
      const int kvh = i / head_dim, e = i % head_dim;
      float v[N];
      Wide<T>::load(row + (size_t)(nq + nkv) * head_dim + i, v);
      Wide<T>::store(v_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim + e, v);
    }
  }
}

// The same with eight-byte accesses (four elements), for head sizes that are a multiple of 8 only.
template <typename T>
__global__ void rope_cache_write_vec4_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                             T* __restrict__ k_pages, T* __restrict__ v_pages, int nq, int nkv,
                                             int head_dim, int page_size, int write_kv) {
  // Positions and slots are the step's metadata and the frequencies are constants: the angles are
  // ready before the kernel that produces qkv has finished.
  extern __shared__ float trig[];            // cos[half], sin[half]
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], trig + half + j, trig + j);
  const int slot = (write_kv && slots) ? slots[t] : -1;
  __syncthreads();
  chain_wait();
  const int row_width = (nq + 2 * nkv) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const int page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? slot % page_size : 0;
  const int per_head = half / 4;              // items per rotated head
  const int rot_items = (nq + nkv) * per_head;
  const int v_items = slot >= 0 ? nkv * head_dim / 4 : 0;
  const int stride = gridDim.y * blockDim.x;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < rot_items + v_items; w += stride) {
    if (w < rot_items) {
      const int head = w / per_head, j = (w % per_head) * 4;
      if (head >= nq && slot < 0) continue;
      T* x = row + (size_t)head * head_dim;
      float a[4], b[4], lo[4], hi[4];
      Pack4<T>::load(x + j, a);
      Pack4<T>::load(x + j + half, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        rotate_pair(a[i], b[i], trig[j + i], trig[half + j + i], lo[i], hi[i]);
      }
      T* dst = x;
      if (head >= nq) dst = k_pages + (((size_t)page * nkv + (head - nq)) * page_size + offset) * head_dim;
      Pack4<T>::store(dst + j, lo);
      Pack4<T>::store(dst + j + half, hi);
    } else {
      const int i = (w - rot_items) * 4;
      const int kvh = i / head_dim, e = i % head_dim;
      float v[4];
      Pack4<T>::load(row + (size_t)(nq + nkv) * head_dim + i, v);
      Pack4<T>::store(v_pages + (((size_t)page * nkv + kvh) * page_size + offset) * head_dim + e, v);
    }
  }
}

// Whether every row of qkv and every head inside it starts on a 16-byte boundary.
static bool row_bytes_16(int nq, int nkv, int head_dim, size_t elem) {
  return ((size_t)(nq + 2 * nkv) * head_dim * elem) % 16 == 0 && ((size_t)head_dim * elem) % 32 == 0;
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
  if (rot_dim == head_dim && head_dim % 8 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)k_pages & 15) &&
      !((uintptr_t)v_pages & 15)) {
    const bool wide = head_dim % (2 * Wide<elem_t>::N) == 0 && row_bytes_16(nq, nkv, head_dim, sizeof(elem_t));
    const int per = wide ? Wide<elem_t>::N : 4;
    const int items = (nq + nkv) * head_dim / (2 * per) + nkv * head_dim / per;
    int y = (items + 127) / 128;
    const int want = (sm_count() * 8 + n_tokens - 1) / n_tokens;      // enough blocks for every SM
    if (y > want) y = want;
    if (y < 1) y = 1;
    if (wide) {
      launch_chained(rope_cache_write_wide_kernel<elem_t>, dim3(dim3(n_tokens, y)), dim3(128), head_dim * sizeof(float), (cudaStream_t)stream,
          (elem_t*)qkv, positions, inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, page_size, write_kv);
      return check_launch("rope_cache_write");
    }
    launch_chained(rope_cache_write_vec4_kernel<elem_t>, dim3(dim3(n_tokens, y)), dim3(128), head_dim * sizeof(float), (cudaStream_t)stream, 
        (elem_t*)qkv, positions, inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, page_size,
        write_kv);
    return check_launch("rope_cache_write");
  }
  launch_chained(rope_cache_write_kernel<elem_t>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (elem_t*)qkv, positions,
      inv_freq, slots, (elem_t*)k_pages, (elem_t*)v_pages, nq, nkv, head_dim, rot_dim, page_size, write_kv);
  return check_launch("rope_cache_write");
}

// ---------------------------------------------------------------------------------------------
// SwiGLU gate: out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], computed in float.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  chain_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx % inter);
  const T* row = gate_up + t * 2 * (size_t)inter;
  const float g = Elem<T>::load(row + i), u = Elem<T>::load(row + inter + i);
  Elem<T>::store(out + idx, silu_mul(g, u));
}

template <typename T> struct Vec16;   // 16-byte groups
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) { load4(p, v); }
  static __device__ __forceinline__ void store(float* p, const float* v) { Pack4<float>::store(p, v); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) { load8(p, v); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    Pack4<__nv_bfloat16>::store(p, v);
    Pack4<__nv_bfloat16>::store(p + 4, v + 4);
  }
};

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t groups) {
  chain_wait();
  constexpr int N = Vec16<T>::N;
  const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= groups) return;
  const int per_row = inter / N;
  const size_t t = gidx / per_row;
  const int i = (int)(gidx % per_row) * N;
  const T* row = gate_up + t * 2 * (size_t)inter;
  float g[N], u[N];
  Vec16<T>::load(row + i, g);
  Vec16<T>::load(row + inter + i, u);
#pragma unroll
  for (int j = 0; j < N; ++j) g[j] = silu_mul(g[j], u[j]);
  Vec16<T>::store(out + t * (size_t)inter + i, g);
}

ERB_EXPORT int erb_swiglu(const void* gate_up, void* out, int n_tokens, int inter, void* stream) {
  if (n_tokens <= 0) return ERB_OK;
  if (inter <= 0) return fail(ERB_ERR_ARG, "swiglu: bad intermediate size");
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  if (inter % Vec16<elem_t>::N == 0 && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15)) {
    const size_t groups = total / Vec16<elem_t>::N;
    launch_chained(swiglu_vec_kernel<elem_t>, dim3((unsigned)((groups + threads - 1) / threads)), dim3(threads), 0, (cudaStream_t)stream, 
        (const elem_t*)gate_up, (elem_t*)out, inter, groups);
    return check_launch("swiglu");
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  launch_chained(swiglu_kernel<elem_t>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (const elem_t*)gate_up, (elem_t*)out,
                                                                     inter, total);
  return check_launch("swiglu");
}

// Rows of a float matrix gathered and cast to T (the rows whose logits are wanted, when the
// stack ends without a norm).
template <typename T>
__global__ void gather_cast_kernel(const float* __restrict__ src, T* __restrict__ dst,
                                   const int* __restrict__ rows, int width) {
  chain_wait();
  const int o = blockIdx.x;
  const float* s = src + (size_t)(rows ? rows[o] : o) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) Elem<T>::store(dst + (size_t)o * width + i, s[i]);
}

ERB_EXPORT int erb_gather_cast(const float* src, void* dst, const int* rows, int n_rows, int width,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  launch_chained(gather_cast_kernel<elem_t>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, src, (elem_t*)dst, rows, width);
  return check_launch("gather_cast");
}

// ---------------------------------------------------------------------------------------------
// Token ids that are still on the device: an id t < 0 in `ids` stands for row -t - 1 of `fed`, the
// tokens the sampler wrote for the step before (the host launches the next step before it has read
// them).  A row outside `fed` leaves the id negative, which the embedding kernel then flags.
// ---------------------------------------------------------------------------------------------
__global__ void resolve_ids_kernel(int* __restrict__ ids, int n, const int* __restrict__ fed, int n_fed) {
  chain_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const int id = ids[t];
  if (id < 0 && -id - 1 < n_fed) ids[t] = fed[-id - 1];
}

ERB_EXPORT int erb_resolve_ids(int* ids, int n, const int* fed, int n_fed, void* stream) {
  if (n <= 0) return ERB_OK;
  if (!ids || !fed || n_fed <= 0) return fail(ERB_ERR_ARG, "resolve_ids: no buffer of fed-back tokens");
  launch_chained(resolve_ids_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, (cudaStream_t)stream, ids, n, fed, n_fed);
  return check_launch("resolve_ids");
}
