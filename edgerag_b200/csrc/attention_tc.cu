// Decode attention (one new token per sequence) for bfloat16: keys and values streamed from the cache
// pages by the asynchronous copy engines.  Two kernels share the split-KV scheme and the scratch layout
// of the general kernel: one for a single query head per kv head (CUDA cores, bulk copies), one for
// grouped query heads (tensor cores, TMA tensor copies).
#include <stdarg.h>
#include <stdio.h>

#undef ERB_ELEM
#define ERB_ELEM 1
#include "tc_common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

// =============================================================================================
// Decode attention (one new token per sequence) streamed with bulk asynchronous copies.
//
// A block owns one (split of keys, kv head, sequence) and all query heads of that kv head's group.
// The keys and values of its split arrive in shared memory through cp.async.bulk copies of whole
// page segments (one contiguous run of rows per page), kStages stages deep, each stage signalled by
// an mbarrier with a transaction count; four warps consume a stage while the next ones are in
// flight, so the bytes in flight per SM are set by the pipeline depth, not by registers.
// Inside a stage a key is handled by D/8 lanes (16 bytes each); the dot product is finished with
// shuffles and every lane keeps the running max, denominator and 8 accumulators of its slice.
// Partial results go to the same scratch layout as the general kernel; a combine kernel merges the
// splits in order.  bfloat16, head size 32, 64 or 128.
// =============================================================================================
namespace {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kStages = 3;
constexpr int kMaxGroup = 8;          // query heads per kv head handled in one pass
constexpr int kKeysPerGroup = 4;      // keys a lane group handles per stage (independent chains)

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Eight bfloat16 values (one 16-byte chunk of shared memory) as floats: a shift and a mask per pair.
__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

constexpr int kCombineMaxSplits = 64;     // splits of one sequence that a merge takes
constexpr int kMergeWarps = 9;            // warps of the largest block that merges (eight and a copy warp)

// The merge of a (sequence, head group)'s splits by the block that finishes last among them, in place
// of a second kernel.  Every block adds one to the group's counter after its partial results are
// visible device-wide; the block that sees n_splits - 1 there is the last, puts the counter back to
// zero (so the array stays zero between launches) and merges: per query head the weights of the
// splits from their maxima (log2 domain), then every output element as a sum over the splits in
// their order.  The result therefore does not depend on which block came last.  A block that gave
// up on a wait does not count, so after a flagged status the host zeroes the counters.
template <int D>
__device__ __forceinline__ void merge_splits_if_last(int* counter, const float* part_acc, const float* part_ml,
                                                     size_t head0, int n_heads, int n_splits, int max_splits,
                                                     __nv_bfloat16* o) {
  __shared__ int s_last;
  __shared__ float s_w[kMergeWarps][kCombineMaxSplits];     // the splits' weights, per warp
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int last = atomicAdd(counter, 1) == n_splits - 1;
    if (last) atomicExch(counter, 0);
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  if (warp >= kMergeWarps) return;
  float* w = s_w[warp];
  for (int h = warp; h < n_heads; h += min(n_warps, kMergeWarps)) {
    const size_t base = (head0 + h) * max_splits;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (lane < n_splits) { m0 = __ldcg(part_ml + (base + lane) * 2); l0 = __ldcg(part_ml + (base + lane) * 2 + 1); }
    if (lane + 32 < n_splits) { m1 = __ldcg(part_ml + (base + lane + 32) * 2); l1 = __ldcg(part_ml + (base + lane + 32) * 2 + 1); }
    const float m = warp_max(fmaxf(m0, m1));
    const float w0 = lane < n_splits ? exp2f(m0 - m) : 0.f, w1 = lane + 32 < n_splits ? exp2f(m1 - m) : 0.f;
    w[lane] = w0;
    w[lane + 32] = w1;
    const float inv = 1.f / warp_sum(l0 * w0 + l1 * w1);
    __syncwarp();
    // A lane owns D / 32 neighbouring elements, so that a split costs it one load and many are in flight.
    constexpr int V = D / 32;
    float sum[V];
#pragma unroll
    for (int i = 0; i < V; ++i) sum[i] = 0.f;
    const float* src = part_acc + base * D + lane * V;
#pragma unroll 8
    for (int sp = 0; sp < n_splits; ++sp) {
      float x[V];
      if constexpr (V == 4) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * D));
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
      } else if constexpr (V == 2) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(src + (size_t)sp * D));
        x[0] = v.x; x[1] = v.y;
      } else {
        x[0] = __ldcg(src + (size_t)sp * D);
      }
#pragma unroll
      for (int i = 0; i < V; ++i) sum[i] += x[i] * w[sp];
    }
#pragma unroll
    for (int i = 0; i < V; ++i) o[(size_t)h * D + lane * V + i] = __float2bfloat16_rn(sum[i] * inv);
    __syncwarp();
  }
}

template <int D, int R>   // head size; query heads per kv head (1..kMaxGroup)
__global__ void __launch_bounds__(kDecThreads)
attention_decode_bulk_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride,
                             const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                             const int* __restrict__ block_tables, int max_pages,
                             const int* __restrict__ token_of_seq, const int* __restrict__ positions,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, int max_splits, int nq,
                             int nkv, int page_size, int split_keys, float scale_log2, int hg,
                             __nv_bfloat16* __restrict__ out, int out_row_stride, int* __restrict__ status,
                             int* __restrict__ counters) {
  // Everything up to chain_wait() below reads only what earlier steps or the host wrote (the batch's
  // metadata, keys and values of earlier tokens), so it runs while the kernel before this one (the
  // one that rotates q and writes this step's keys and values) is still at work.
  // hg: kv heads handled by this block.  The rows of hg neighbouring heads of one page are contiguous
  // in the cache, so a block that takes them together copies hg * page_size rows in one piece; with
  // small pages that is what keeps the copies long enough for the memory system.
  constexpr int LPK = D / 8;                              // lanes per key (16 bytes each)
  constexpr int GPW = 32 / LPK;                           // lane groups per warp
  constexpr int STAGE_ROWS = kDecWarps * GPW * kKeysPerGroup;   // (key, head) rows per stage: 16 KB of K and of V
  constexpr int ROW = D * 2;                              // bytes per key row
  constexpr uint32_t STAGE_BYTES = STAGE_ROWS * ROW;
  const int STAGE_KEYS = STAGE_ROWS / hg;                  // keys of each head per stage
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  uint8_t* smem = smem_raw + (base - raw);
  // layout: K stages | V stages | barriers | merge area | page ids
  const uint32_t sK = base, sV = base + kStages * STAGE_BYTES, sBar = sV + kStages * STAGE_BYTES;
  float* merge = reinterpret_cast<float*>(smem + 2 * kStages * STAGE_BYTES + 64);   // [warps][R][D + 2]
  int* s_pages = reinterpret_cast<int*>(merge + kDecWarps * R * (D + 2));

  const int split = blockIdx.x, kvh0 = blockIdx.y * hg, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warps_per_head = kDecWarps / hg;
  const int hh = warp / warps_per_head;                    // which head of the group this warp serves
  const int kvh = kvh0 + hh;
  // The last group may hold fewer heads than hg (a head count that hg does not divide): the stage
  // keeps its layout for hg heads, the copies bring the heads there are, the other warps idle.
  const int hg_here = min(hg, nkv - kvh0);
  const bool serves = hh < hg_here;
  const int t = token_of_seq[seq];
  const int pos = positions[t];
  const int begin = split * split_keys;
  const int end = min(pos + 1, begin + split_keys);
  if (begin >= end) return;
  const int* bt = block_tables + (size_t)seq * max_pages;
  const int n_tiles = (end - begin + STAGE_KEYS - 1) / STAGE_KEYS;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sBar + 8 * s));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The block table entries of the split, fetched by all threads at once: the thread that issues
  // the copies must not wait on a global load per page.
  const int first_page = begin / page_size;
  const int n_pages = (end - 1) / page_size - first_page + 1;
  for (int i = tid; i < n_pages; i += kDecThreads) s_pages[i] = bt[first_page + i];
  __syncthreads();

  auto issue = [&](int tile) {   // thread 0 only
    const int s = tile % kStages;
    const int kb = begin + tile * STAGE_KEYS, ke = min(end, kb + STAGE_KEYS);
    const uint32_t bar = sBar + 8 * s;
    if (hg == 1) {
      // one head: copy exactly the visible keys, one run per page
      mbar_expect(bar, (uint32_t)(ke - kb) * ROW * 2);
      int k = kb;
      while (k < ke) {
        const int page = s_pages[k / page_size - first_page], off = k % page_size;
        const int n = min(page_size - off, ke - k);
        const size_t src = (((size_t)page * nkv + kvh0) * page_size + off) * D;
        const uint32_t dst = (uint32_t)(s * STAGE_BYTES + (k - kb) * ROW);
        bulk_copy(sK + dst, k_pages + src, (uint32_t)n * ROW, bar);
        bulk_copy(sV + dst, v_pages + src, (uint32_t)n * ROW, bar);
        k += n;
      }
    } else {
      // hg heads: whole pages (kb is a multiple of page_size), hg * page_size rows per copy
      const int n_pg = (ke - kb + page_size - 1) / page_size;
      const uint32_t slot_bytes = (uint32_t)(hg * page_size) * ROW;         // room of one page in the stage
      const uint32_t chunk_bytes = (uint32_t)(hg_here * page_size) * ROW;   // what one page brings
      mbar_expect(bar, (uint32_t)n_pg * chunk_bytes * 2);
      for (int j = 0; j < n_pg; ++j) {
        const int page = s_pages[kb / page_size + j - first_page];
        const size_t src = ((size_t)page * nkv + kvh0) * page_size * D;
        const uint32_t dst = (uint32_t)(s * STAGE_BYTES) + (uint32_t)j * slot_bytes;
        bulk_copy(sK + dst, k_pages + src, chunk_bytes, bar);
        bulk_copy(sV + dst, v_pages + src, chunk_bytes, bar);
      }
    }
  };
  // Tiles that end before the page of the new token hold nothing this step has written.
  const int old_end = (pos / page_size) * page_size;
  int issued = 0;
  if (tid == 0) {
    while (issued < kStages && issued < n_tiles && min(end, begin + (issued + 1) * STAGE_KEYS) <= old_end) issue(issued++);
  }
  chain_wait();
  if (tid == 0) {
    for (int i = issued; i < kStages && i < n_tiles; ++i) issue(i);
  }

  // This lane's slice of every query head of the group, pre-multiplied by scale * log2(e).
  const int sub = lane / LPK, chunk = lane % LPK;
  float qr[R][8];
#pragma unroll
  for (int g = 0; g < R; ++g) {
    const __nv_bfloat16* qp = q + (size_t)t * q_row_stride + (size_t)((serves ? kvh : kvh0) * R + g) * D + chunk * 8;
    float tmp[8];
    load8(qp, tmp);
#pragma unroll
    for (int i = 0; i < 8; ++i) qr[g][i] = tmp[i] * scale_log2;
  }
  float m_run[R], l_run[R], acc[R][8];
#pragma unroll
  for (int g = 0; g < R; ++g) {
    m_run[g] = -INFINITY; l_run[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  bool ok = true;
  // this lane group's first key (of its head) inside a stage, and where that row sits in the stage:
  // with hg > 1 a stage holds pages one after the other, each page holding its hg heads in turn
  const int key_in_stage = ((warp % warps_per_head) * GPW + sub) * kKeysPerGroup;
  const int row_offset = (hg == 1) ? key_in_stage * ROW
                                   : ((key_in_stage / page_size) * hg * page_size + hh * page_size +
                                      key_in_stage % page_size) * ROW;
  const uint32_t group_mask = (LPK == 32 ? 0xffffffffu : ((1u << LPK) - 1u)) << (sub * LPK);   // lanes of this key group
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kStages;
    if (ok && !mbar_wait(sBar + 8 * s, (tile / kStages) & 1)) ok = false;
    const int n_here = min(end - (begin + tile * STAGE_KEYS), STAGE_KEYS);
    if (ok && serves && key_in_stage < n_here) {
      const uint8_t* kt = smem + s * STAGE_BYTES + row_offset + chunk * 16;
      const uint8_t* vt = kt + kStages * STAGE_BYTES;
      uint4 kraw[kKeysPerGroup];
#pragma unroll
      for (int u = 0; u < kKeysPerGroup; ++u) kraw[u] = *reinterpret_cast<const uint4*>(kt + u * ROW);
      float sc[R][kKeysPerGroup];
#pragma unroll
      for (int u = 0; u < kKeysPerGroup; ++u) {
        float kf[8];
        unpack8(kraw[u], kf);
#pragma unroll
        for (int g = 0; g < R; ++g) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) d = fmaf(qr[g][i], kf[i], d);
          sc[g][u] = d;
        }
      }
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) {
#pragma unroll
        for (int g = 0; g < R; ++g) {
#pragma unroll
          for (int u = 0; u < kKeysPerGroup; ++u) sc[g][u] += __shfl_xor_sync(group_mask, sc[g][u], o);
        }
      }
      uint4 vraw[kKeysPerGroup];
#pragma unroll
      for (int u = 0; u < kKeysPerGroup; ++u) vraw[u] = *reinterpret_cast<const uint4*>(vt + u * ROW);
      float p[R][kKeysPerGroup];
#pragma unroll
      for (int g = 0; g < R; ++g) {
        float m_new = m_run[g];
#pragma unroll
        for (int u = 0; u < kKeysPerGroup; ++u) {
          if (key_in_stage + u >= n_here) sc[g][u] = -INFINITY;     // keys past the end of the split
          m_new = fmaxf(m_new, sc[g][u]);
        }
        // key_in_stage < n_here: at least one key is real, so m_new is finite
        const float a = exp2f(m_run[g] - m_new);
        float sum = 0.f;
#pragma unroll
        for (int u = 0; u < kKeysPerGroup; ++u) { p[g][u] = exp2f(sc[g][u] - m_new); sum += p[g][u]; }
        l_run[g] = l_run[g] * a + sum;
        m_run[g] = m_new;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] *= a;
      }
#pragma unroll
      for (int u = 0; u < kKeysPerGroup; ++u) {
        float vf[8];
        unpack8(vraw[u], vf);
        if (key_in_stage + u >= n_here) {                           // unwritten rows may hold anything
#pragma unroll
          for (int i = 0; i < 8; ++i) vf[i] = 0.f;
        }
#pragma unroll
        for (int g = 0; g < R; ++g) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p[g][u], vf[i], acc[g][i]);
        }
      }
    }
    __syncthreads();                                        // everyone is done with stage s
    if (tid == 0 && ok && tile + kStages < n_tiles) issue(tile + kStages);
  }

  // Merge the lane groups of each warp (lanes that share `chunk`), then the warps.
#pragma unroll
  for (int g = 0; g < R; ++g) {
    float m = m_run[g];
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float f = (m_run[g] == -INFINITY) ? 0.f : exp2f(m_run[g] - m);
    float l = l_run[g] * f;
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = acc[g][i] * f;
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      acc[g][i] = a;
    }
    float* w = merge + (warp * R + g) * (D + 2);
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[chunk * 8 + i] = acc[g][i];
      if (chunk == 0) { w[D] = m; w[D + 1] = l; }
    }
  }
  __syncthreads();
  if (!ok) {
    if (tid == 0) atomicCAS(status, 0, 2000000 + (int)blockIdx.x);
    return;
  }
  for (int idx = tid; idx < hg_here * R * D; idx += kDecThreads) {
    const int head = idx / (R * D), g = (idx / D) % R, d = idx % D;
    const int w0 = head * warps_per_head;
    float m = -INFINITY;
    for (int w = w0; w < w0 + warps_per_head; ++w) m = fmaxf(m, merge[(w * R + g) * (D + 2) + D]);
    float sum = 0.f, l = 0.f;
    for (int w = w0; w < w0 + warps_per_head; ++w) {
      const float mw = merge[(w * R + g) * (D + 2) + D];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      sum += merge[(w * R + g) * (D + 2) + d] * f;
      l += merge[(w * R + g) * (D + 2) + D + 1] * f;
    }
    if (max_splits == 1) {      // the only split: this is the result (what the combine kernel would make of it)
      out[(size_t)t * out_row_stride + (size_t)((kvh0 + head) * R + g) * D + d] = __float2bfloat16_rn(sum * (1.f / l));
      continue;
    }
    const size_t slot = ((size_t)seq * nq + (kvh0 + head) * R + g) * max_splits + split;
    part_acc[slot * D + d] = sum;
    if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
  }
  if (max_splits > 1 && counters)
    merge_splits_if_last<D>(counters + (size_t)seq * gridDim.y + blockIdx.y, part_acc, part_ml,
                            (size_t)seq * nq + (size_t)kvh0 * R, hg_here * R, min(pos / split_keys + 1, max_splits), max_splits,
                            out + (size_t)t * out_row_stride + (size_t)kvh0 * R * D);
}

// Merges the splits of each (sequence, head).  The partial maxima are in the log2 domain.  The
// weights of the splits are computed by the first lanes in parallel; every output element is then
// a sum over the splits in their order.
__global__ void __launch_bounds__(64)
attention_decode_bulk_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                     const int* __restrict__ token_of_seq, const int* __restrict__ positions,
                                     __nv_bfloat16* __restrict__ out, int out_row_stride, int max_splits,
                                     int nq, int head_dim, int split_keys) {
  chain_wait();
  __shared__ float s_w[kCombineMaxSplits];
  __shared__ float s_red[2];
  const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  const int t = token_of_seq[seq];
  const int n_splits = min(positions[t] / split_keys + 1, max_splits);   // never beyond what the split kernel wrote
  const size_t base = ((size_t)seq * nq + h) * max_splits;
  float m_i = -INFINITY, l_i = 0.f;
  if (tid < n_splits) { m_i = part_ml[(base + tid) * 2]; l_i = part_ml[(base + tid) * 2 + 1]; }
  float m = warp_max(m_i);
  if ((tid & 31) == 0) s_red[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(s_red[0], s_red[1]);
  const float w_i = (tid < n_splits) ? exp2f(m_i - m) : 0.f;
  if (tid < kCombineMaxSplits) s_w[tid] = w_i;
  float l = warp_sum(l_i * w_i);
  __syncthreads();
  if ((tid & 31) == 0) s_red[tid >> 5] = l;
  __syncthreads();
  const float inv = 1.f / (s_red[0] + s_red[1]);
  __nv_bfloat16* o = out + (size_t)t * out_row_stride + (size_t)h * head_dim;
  for (int d = tid; d < head_dim; d += 64) {
    float sum = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) sum += part_acc[(base + s) * head_dim + d] * s_w[s];
    o[d] = __float2bfloat16_rn(sum * inv);
  }
}

// Heads per block of the bulk decode kernel: enough neighbouring kv heads that one page's rows make
// a copy of about 8 KB, as long as whole pages tile a stage and the split.  A head count that this
// does not divide gets one block for all its heads when they are at most 8 and their copy stays
// within 16 KB (5 heads of 64 with 16-token pages: 10 KB copies instead of 2 KB ones), else a last
// group with the heads that are left.
// `want` > 0 asks for that many heads per block (a power of two that passes the same checks; 1 always
// does): fewer heads per block give more and shorter blocks, which is what a small batch of short
// contexts needs.  The answer is 0 when `want` cannot be had.
int decode_head_group(int nkv, int head_dim, int page_size, int split_keys, int want = 0) {
  const int stage_rows = kDecWarps * (32 / (head_dim / 8)) * kKeysPerGroup;
  auto fits = [&](int hg) { return hg <= kDecWarps && (stage_rows / hg) % page_size == 0 && stage_rows / hg >= page_size; };
  if (want == 1) return 1;
  if (want > 1) return (want & (want - 1)) == 0 && split_keys % page_size == 0 && fits(want) && want < 2 * nkv ? want : 0;
  if (split_keys % page_size) return 1;
  int hg = 1;
  while (hg * 2 * page_size * head_dim * 2 <= 8192 && fits(hg * 2) && hg < nkv) hg *= 2;
  if (nkv % hg) {
    int all = 1;
    while (all < nkv) all *= 2;
    if (all > hg && fits(all) && nkv * page_size * head_dim * 2 <= 16384) hg = all;
  }
  return hg;
}

template <int D, int R>
int launch_decode_bulk(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                       const int* block_tables, int max_pages, const int* token_of_seq, const int* positions,
                       float* part_acc, float* part_ml, int max_splits, int n_seqs, int nq, int nkv, int page_size,
                       int split_keys, float scale_log2, void* out, int out_row_stride, int* status, int* counters, int head_group,
                       cudaStream_t s) {
  const int hg = decode_head_group(nkv, D, page_size, split_keys, head_group);
  if (hg <= 0) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: %d heads per block with pages of %d and splits of %d", head_group, page_size, split_keys);
  constexpr int STAGE_BYTES = kDecWarps * (32 / (D / 8)) * kKeysPerGroup * D * 2;
  const size_t smem = 2 * kStages * STAGE_BYTES + 64 + (size_t)kDecWarps * R * (D + 2) * sizeof(float) + 128 +
                      (size_t)(split_keys / page_size + 2) * sizeof(int);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: split of %d keys in pages of %d", split_keys, page_size);
  auto kern = attention_decode_bulk_kernel<D, R>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_decode_bulk: %s", cudaGetErrorString(e));
    configured = smem;
  }
  launch_chained(kern, dim3(dim3(max_splits, (nkv + hg - 1) / hg, n_seqs)), dim3(kDecThreads), smem, s, (const __nv_bfloat16*)q, q_row_stride,
      (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_tables, max_pages, token_of_seq, positions,
      part_acc, part_ml, max_splits, nq, nkv, page_size, split_keys, scale_log2, hg, (__nv_bfloat16*)out, out_row_stride, status, counters);
  return check_launch("attention_decode_bulk");
}

template <int D>
int dispatch_group(int r, const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                   const int* block_tables, int max_pages, const int* token_of_seq, const int* positions,
                   float* part_acc, float* part_ml, int max_splits, int n_seqs, int nq, int nkv, int page_size,
                   int split_keys, float scale_log2, void* out, int out_row_stride, int* status, int* counters, int head_group,
                   cudaStream_t s) {
#define ERB_R(RR)                                                                                              \
  case RR: return launch_decode_bulk<D, RR>(q, q_row_stride, k_pages, v_pages, block_tables, max_pages,        \
                                            token_of_seq, positions, part_acc, part_ml, max_splits, n_seqs, nq, \
                                            nkv, page_size, split_keys, scale_log2, out, out_row_stride,       \
                                            status, counters, head_group, s);
  switch (r) { ERB_R(1) ERB_R(2) ERB_R(3) ERB_R(4) ERB_R(5) ERB_R(6) ERB_R(7) ERB_R(8) }
#undef ERB_R
  return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: %d query heads per kv head (at most %d)", r, kMaxGroup);
}

}  // namespace

// =============================================================================================
// Decode attention for grouped query heads (2 to 8 query heads per kv head) on tensor cores.
//
// With several query heads per kv head the CUDA-core kernel above does its arithmetic once per
// query head and key and falls behind the memory (3.4 TB/s at three heads per kv head).  Here the
// query heads of a kv head are the rows of an mma.sync.m16n8k16 tile, so a key costs the same
// whatever their number:
//
//   S[heads x 8 keys]   = Q[heads x 64] K^T       A = Q from registers, B = K rows via ldmatrix
//   O[heads x 64]      += P[heads x 16 keys] V    A = P from the S registers, B = V via ldmatrix.trans
//
// The block structure is that of the kernel above: a block owns one (split of keys, group of hg
// neighbouring kv heads, sequence); whole pages arrive in stages of 128 rows of K and of V, three
// stages deep, completion counted by an mbarrier; a warp serves 16 keys of one kv head per stage;
// partial results of warps and splits are merged exactly as above.  The difference in the data
// path: pages are brought in by TMA tensor copies (cp.async.bulk.tensor.2d) through tensor maps
// over the page pools with the 128-byte swizzle, so that the ldmatrix reads of 8 rows x 16 bytes
// touch all banks.  bfloat16, head size 64, pages of a multiple of 8 tokens.
// =============================================================================================
namespace {

constexpr int kGqaStageRows = 128;                         // rows (key, head) of K and of V per stage
constexpr uint32_t kGqaStageBytes = kGqaStageRows * 128;   // 16 KB
constexpr int kGqaStages = 3;
constexpr int kGqaMaxHeads = 8;                            // query heads per kv head (rows 0..7 of the tile)
constexpr int kGqaThreads = kDecThreads + 32;               // eight multiplying warps and a copy warp

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// d += a * b, a: 16 x 16 (rows 8..15 are zero: a1 = a3 = 0), b: 16 x 8
__device__ __forceinline__ void mma_heads(float* d, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(kGqaThreads)
attention_decode_gqa_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __grid_constant__ CUtensorMap map_k_last, const __grid_constant__ CUtensorMap map_v_last,
                            const __nv_bfloat16* __restrict__ q, int q_row_stride,
                            const int* __restrict__ block_tables, int max_pages,
                            const int* __restrict__ token_of_seq, const int* __restrict__ positions,
                            float* __restrict__ part_acc, float* __restrict__ part_ml, int max_splits, int nq,
                            int nkv, int page_size, int split_keys, float scale_log2, int hg,
                            __nv_bfloat16* __restrict__ out, int out_row_stride, int* __restrict__ status,
                            int* __restrict__ counters) {
  constexpr int D = 64;
  const int R = nq / nkv;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;            // the swizzle repeats every 1024 bytes
  uint8_t* smem = smem_raw + (base - raw);
  // layout: K stages | V stages | barriers | merge area | page ids
  const uint32_t sK = base, sV = base + kGqaStages * kGqaStageBytes, sBar = sV + kGqaStages * kGqaStageBytes;
  const uint32_t sEmpty = sBar + 8 * kGqaStages;           // consumers -> copy warp: the stage is free again
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + 2 * kGqaStages * kGqaStageBytes + 56);
  float* merge = reinterpret_cast<float*>(smem + 2 * kGqaStages * kGqaStageBytes + 64);   // [warps][R][D + 2]
  int* s_pages = reinterpret_cast<int*>(merge + kDecWarps * R * (D + 2));

  const int split = blockIdx.x, kvh0 = blockIdx.y * hg, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int warps_per_head = kDecWarps / hg;
  const int hh = warp / warps_per_head, ws = warp % warps_per_head;
  const int hg_here = min(hg, nkv - kvh0);
  const bool serves = hh < hg_here;
  const int stage_keys = kGqaStageRows / hg;               // keys of each head per stage
  const int t = token_of_seq[seq];
  const int pos = positions[t];
  const int begin = split * split_keys;
  const int end = min(pos + 1, begin + split_keys);
  if (begin >= end) return;
  const int* bt = block_tables + (size_t)seq * max_pages;
  const int n_tiles = (end - begin + stage_keys - 1) / stage_keys;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kGqaStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sBar + 8 * s));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sEmpty + 8 * s), "n"(kDecWarps));
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int first_page = begin / page_size;
  const int n_pages = (end - 1) / page_size - first_page + 1;
  for (int i = tid; i < n_pages; i += kGqaThreads) s_pages[i] = bt[first_page + i];
  __syncthreads();
  // A wait that gives up when its own limit runs out or when another thread of the block has given up.
  auto wait_for = [&](uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
      uint32_t done;
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}\n"
          : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) return true;
      if (*s_abort) return false;
    }
    *s_abort = 1;
    return false;
  };

  const CUtensorMap* mk = hg_here == hg ? &map_k : &map_k_last;
  const CUtensorMap* mv = hg_here == hg ? &map_v : &map_v_last;
  const uint32_t page_slot = (uint32_t)(hg * page_size) * 128u;          // room of one page in a stage
  const uint32_t page_bytes = (uint32_t)(hg_here * page_size) * 128u;    // what one page brings
  auto issue = [&](int tile) {   // one lane of the copy warp: whole pages, hg_here * page_size rows per copy
    const int s = tile % kGqaStages;
    const int kb = begin + tile * stage_keys, ke = min(end, kb + stage_keys);
    const uint32_t bar = sBar + 8 * s;
    const int n_pg = (ke - kb + page_size - 1) / page_size;
    mbar_expect(bar, (uint32_t)n_pg * page_bytes * 2);
    for (int j = 0; j < n_pg; ++j) {
      const int page = s_pages[kb / page_size + j - first_page];
      const int row = (page * nkv + kvh0) * page_size;
      const uint32_t dst = (uint32_t)s * kGqaStageBytes + (uint32_t)j * page_slot;
      tma_load_rows(sK + dst, mk, row, bar);
      tma_load_rows(sV + dst, mv, row, bar);
    }
  };
  if (warp == kDecWarps) {
    // ---- the copy warp: one lane asks for tile after tile, as soon as the stage it goes into is free ----
    // Tiles that end before the page of the new token hold nothing this step has written: they are
    // asked for before the wait for the kernel that writes this step's keys and rotates q.
    if (lane == 0) {
      const int old_end = (pos / page_size) * page_size;
      bool waited = false;
      for (int tile = 0; tile < n_tiles; ++tile) {
        if (!waited && min(end, begin + (tile + 1) * stage_keys) > old_end) { chain_wait(); waited = true; }
        if (tile >= kGqaStages && !wait_for(sEmpty + 8 * (tile % kGqaStages), ((tile / kGqaStages) - 1) & 1)) break;
        issue(tile);
      }
      if (!waited) chain_wait();
    }
    __syncwarp();
  }
  chain_wait();

  // Q of this warp's kv head as the A operand: row g = lane / 4 is query head g of the group.
  const int g = lane >> 2, j = lane & 3;
  uint32_t qa[4][2];
  {
    const bool real = serves && g < R;
    const __nv_bfloat16* qp = q + (size_t)t * q_row_stride + (size_t)((real ? (kvh0 + hh) * R + g : 0)) * D;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      qa[ks][0] = real ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * j) : 0u;
      qa[ks][1] = real ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * j + 8) : 0u;
    }
  }
  float o[8][4];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nb][i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;      // of row g; l_run is this lane's share of the row's sum

  // Rows of this warp's two blocks of 8 keys inside a stage: key k of head hh sits in row
  // ((k / page_size) * hg + hh) * page_size + k % page_size.
  const int key0 = ws * 16;
  auto row_of = [&](int k) { return ((k / page_size) * hg + hh) * page_size + k % page_size; };
  const int row_a = row_of(key0), row_b = row_of(key0 + 8);
  const int mi = lane >> 3, ri = lane & 7;   // ldmatrix: this lane gives the address of row ri of matrix mi

  bool ok = true;
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kGqaStages;
    if (warp == kDecWarps) break;                           // the copy warp has nothing to multiply
    if (ok && !wait_for(sBar + 8 * s, (tile / kGqaStages) & 1)) ok = false;
    const int n_here = min(end - (begin + tile * stage_keys), stage_keys);
    if (ok && serves && key0 < n_here) {
      const uint32_t k_st = sK + (uint32_t)s * kGqaStageBytes, v_st = sV + (uint32_t)s * kGqaStageBytes;
      // Rows past the last key may hold anything (unwritten slots, an earlier tile): their scores are
      // masked below, and their values are zeroed here, since 0 * NaN would spoil the product.
      if (key0 + 16 > n_here) {
        for (int k = max(n_here, key0) * 8 + lane; k < (key0 + 16) * 8; k += 32) {
          const int key = k >> 3, chunk = k & 7;
          *reinterpret_cast<uint4*>(smem + (v_st - base) + row_of(key) * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      // S for the two blocks of 8 keys
      float sc[2][4];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int row = (b ? row_b : row_a) + ri;
        sc[b][0] = sc[b][1] = sc[b][2] = sc[b][3] = 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t kf[4];
          ldmatrix_x4(k_st + (uint32_t)row * 128u + (uint32_t)(((half * 4 + mi) ^ ri) << 4), kf);
          mma_heads(sc[b], qa[half * 2][0], qa[half * 2][1], kf[0], kf[1]);
          mma_heads(sc[b], qa[half * 2 + 1][0], qa[half * 2 + 1][1], kf[2], kf[3]);
        }
      }
      // this lane: row g, keys key0 + 8 b + 2 j, + 1
      float m_new = m_run;
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int key = key0 + 8 * b + 2 * j + i;
          sc[b][i] = key < n_here ? sc[b][i] * scale_log2 : -INFINITY;
          m_new = fmaxf(m_new, sc[b][i]);
        }
      m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 1));
      m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, 2));
      // key0 < n_here: the row has at least one real key, so m_new is finite
      const float a = exp2f(m_run - m_new);
      float p[2][2], sum = 0.f;
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 2; ++i) { p[b][i] = exp2f(sc[b][i] - m_new); sum += p[b][i]; }
      l_run = l_run * a + sum;
      m_run = m_new;
      const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]), pa2 = pack_bf16(p[1][0], p[1][1]);
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) { o[nb][0] *= a; o[nb][1] *= a; }
      // O += P V over the 16 keys: matrices (keys 0..7 | 8..15) x (8 values of chunk nb | nb + 1)
#pragma unroll
      for (int nb = 0; nb < 8; nb += 2) {
        uint32_t vf[4];
        const int row = ((mi & 1) ? row_b : row_a) + ri;
        ldmatrix_x4_trans(v_st + (uint32_t)row * 128u + (uint32_t)(((nb + (mi >> 1)) ^ ri) << 4), vf);
        mma_heads(o[nb], pa0, pa2, vf[0], vf[1]);
        mma_heads(o[nb + 1], pa0, pa2, vf[2], vf[3]);
      }
    }
    __syncwarp();                                           // this warp is done with stage s
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sEmpty + 8 * s) : "memory");
  }

  // The row's sum over its four lanes; then this warp's result for its query heads.
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (warp < kDecWarps && g < R) {
    float* w = merge + (warp * R + g) * (D + 2);
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { w[nb * 8 + 2 * j] = o[nb][0]; w[nb * 8 + 2 * j + 1] = o[nb][1]; }
    if (j == 0) { w[D] = m_run; w[D + 1] = l_run; }
  }
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicCAS(status, 0, 2000000 + (int)blockIdx.x);
    return;
  }
  for (int idx = tid; idx < hg_here * R * D; idx += kGqaThreads) {
    const int head = idx / (R * D), gq = (idx / D) % R, d = idx % D;
    const int w0 = head * warps_per_head;
    float m = -INFINITY;
    for (int w = w0; w < w0 + warps_per_head; ++w) m = fmaxf(m, merge[(w * R + gq) * (D + 2) + D]);
    float sum = 0.f, l = 0.f;
    for (int w = w0; w < w0 + warps_per_head; ++w) {
      const float mw = merge[(w * R + gq) * (D + 2) + D];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
      sum += merge[(w * R + gq) * (D + 2) + d] * f;
      l += merge[(w * R + gq) * (D + 2) + D + 1] * f;
    }
    if (max_splits == 1) {      // the only split: this is the result (what the combine kernel would make of it)
      out[(size_t)t * out_row_stride + (size_t)((kvh0 + head) * R + gq) * D + d] = __float2bfloat16_rn(sum * (1.f / l));
      continue;
    }
    const size_t slot = ((size_t)seq * nq + (kvh0 + head) * R + gq) * max_splits + split;
    part_acc[slot * D + d] = sum;
    if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
  }
  if (max_splits > 1 && counters)
    merge_splits_if_last<D>(counters + (size_t)seq * gridDim.y + blockIdx.y, part_acc, part_ml,
                            (size_t)seq * nq + (size_t)kvh0 * R, hg_here * R, min(pos / split_keys + 1, max_splits), max_splits,
                            out + (size_t)t * out_row_stride + (size_t)kvh0 * R * D);
}

}  // namespace

// Whether erb_attention_decode_gqa takes these sizes (bfloat16 is implied).
ERB_EXPORT int erb_attention_decode_gqa_supported(int nq, int nkv, int head_dim, int page_size, int split_keys) {
  if (head_dim != 64 || nq <= 0 || nkv <= 0 || nq % nkv) return 0;
  const int r = nq / nkv;
  if (r < 2 || r > kGqaMaxHeads || page_size <= 0 || page_size % 8 || split_keys <= 0 || split_keys % page_size) return 0;
  const int hg = decode_head_group(nkv, 64, page_size, split_keys);
  return (kGqaStageRows / hg) % page_size == 0 && hg * page_size <= 256 && min(hg, nkv) * page_size <= 256;
}

// Same contract as erb_attention_decode_bulk, for 2 to 8 query heads per kv head of size 64;
// n_pool_pages is the number of pages of k_pages / v_pages (the tensor maps cover the whole pool).
ERB_EXPORT int erb_attention_decode_gqa(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                        int n_pool_pages, const int* block_tables, int max_pages,
                                        const int* token_of_seq, const int* positions, void* out, int out_row_stride,
                                        float* part_acc, float* part_ml, int max_splits, int n_seqs, int nq, int nkv,
                                        int head_dim, int page_size, int split_keys, float scale, int* status,
                                        int* counters, void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  if (!erb_attention_decode_gqa_supported(nq, nkv, head_dim, page_size, split_keys))
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: %d/%d heads of %d, pages of %d, splits of %d", nq, nkv,
                head_dim, page_size, split_keys);
  if (max_splits <= 0 || !part_acc || !part_ml || !status || n_pool_pages <= 0)
    return fail(ERB_ERR_ARG, "attention_decode_gqa: bad arguments");
  if (q_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127))
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: q rows must be 16-byte aligned, pools 128-byte aligned");
  if (n_seqs > 65535 || nkv > 65535) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: grid too large");
  if (max_splits > kCombineMaxSplits)
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: %d splits (at most %d)", max_splits, kCombineMaxSplits);
  if ((unsigned long long)n_pool_pages * nkv * page_size > 0x7fffffffull)
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: pool too large for 32-bit row coordinates");
  const int hg = decode_head_group(nkv, 64, page_size, split_keys);
  const int last = nkv % hg ? nkv % hg : hg;
  const unsigned long long rows = (unsigned long long)n_pool_pages * nkv * page_size;
  CUtensorMap mk, mv, mkl, mvl;
  int rc;
  if ((rc = pool_map(&mk, k_pages, rows, (unsigned)(hg * page_size), "attention_decode_gqa")) || (rc = pool_map(&mv, v_pages, rows, (unsigned)(hg * page_size), "attention_decode_gqa")) ||
      (rc = pool_map(&mkl, k_pages, rows, (unsigned)(last * page_size), "attention_decode_gqa")) || (rc = pool_map(&mvl, v_pages, rows, (unsigned)(last * page_size), "attention_decode_gqa")))
    return rc;
  const int r = nq / nkv;
  const size_t smem = 1024 + 2 * kGqaStages * kGqaStageBytes + 64 + (size_t)kDecWarps * r * (64 + 2) * sizeof(float) + 128 +
                      (size_t)(split_keys / page_size + 2) * sizeof(int);
  if (smem > 200 * 1024) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_gqa: split of %d keys in pages of %d", split_keys, page_size);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_gqa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_decode_gqa: %s", cudaGetErrorString(e));
    configured = smem;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_chained(attention_decode_gqa_kernel, dim3(dim3(max_splits, (nkv + hg - 1) / hg, n_seqs)), dim3(kGqaThreads), smem, s,
                 mk, mv, mkl, mvl, (const __nv_bfloat16*)q, q_row_stride, block_tables, max_pages, token_of_seq, positions,
                 part_acc, part_ml, max_splits, nq, nkv, page_size, split_keys, scale_log2, hg, (__nv_bfloat16*)out, out_row_stride,
                 status, counters);
  // a single split wrote the result itself; with counters the block that finishes last merges the splits
  if ((rc = check_launch("attention_decode_gqa")) || max_splits == 1 || counters) return rc;
  launch_chained(attention_decode_bulk_combine_kernel, dim3(dim3(nq, n_seqs)), dim3(64), 0, s, part_acc, part_ml, token_of_seq, positions,
      (__nv_bfloat16*)out, out_row_stride, max_splits, nq, head_dim, split_keys);
  return check_launch("attention_decode_bulk_combine");
}

// Blocks per sequence and split of erb_attention_decode_bulk (groups of kv heads), for sizing decisions.
ERB_EXPORT int erb_attention_decode_bulk_groups(int nkv, int head_dim, int page_size, int split_keys) {
  if (nkv <= 0 || page_size <= 0 || (head_dim != 32 && head_dim != 64 && head_dim != 128)) return nkv > 0 ? nkv : 1;
  const int hg = decode_head_group(nkv, head_dim, page_size, split_keys);
  return (nkv + hg - 1) / hg;
}

// Heads per block that erb_attention_decode_bulk uses when asked for `want` (0: its own choice); 0 when
// `want` cannot be had with these sizes.
ERB_EXPORT int erb_attention_decode_bulk_head_group(int nkv, int head_dim, int page_size, int split_keys, int want) {
  if (nkv <= 0 || page_size <= 0 || split_keys <= 0 || (head_dim != 32 && head_dim != 64 && head_dim != 128)) return 0;
  return decode_head_group(nkv, head_dim, page_size, split_keys, want);
}

// Same contract as the general decode entry point (scratch provided by the caller, splits at
// absolute multiples of split_keys), for bfloat16 with head_dim 32 / 64 / 128, no window, at most
// 8 query heads per kv head, and page rows that are 16-byte multiples.
ERB_EXPORT int erb_attention_decode_bulk(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                         const int* block_tables, int max_pages, const int* token_of_seq,
                                         const int* positions, void* out, int out_row_stride, float* part_acc,
                                         float* part_ml, int max_splits, int n_seqs, int nq, int nkv, int head_dim,
                                         int page_size, int split_keys, float scale, int* status, int* counters,
                                         int head_group, void* stream) {
  if (n_seqs <= 0) return ERB_OK;
  if (nq <= 0 || nkv <= 0 || nq % nkv) return fail(ERB_ERR_ARG, "attention_decode_bulk: bad head counts");
  if (max_splits <= 0 || split_keys <= 0 || !part_acc || !part_ml || !status || page_size <= 0)
    return fail(ERB_ERR_ARG, "attention_decode_bulk: bad arguments");
  if (q_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: rows must be 16-byte aligned");
  if (n_seqs > 65535 || nkv > 65535) return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: grid too large");
  if (max_splits > kCombineMaxSplits)
    return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: %d splits (at most %d)", max_splits, kCombineMaxSplits);
  const float scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  const int r = nq / nkv;
  int rc;
  switch (head_dim) {
    case 32: rc = dispatch_group<32>(r, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                                     positions, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size, split_keys,
                                     scale_log2, out, out_row_stride, status, counters, head_group, s); break;
    case 64: rc = dispatch_group<64>(r, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                                     positions, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size, split_keys,
                                     scale_log2, out, out_row_stride, status, counters, head_group, s); break;
    case 128: rc = dispatch_group<128>(r, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                                       positions, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size,
                                       split_keys, scale_log2, out, out_row_stride, status, counters, head_group, s); break;
    default: return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: head_dim %d (takes 32, 64, 128)", head_dim);
  }
  // a single split wrote the result itself; with counters the block that finishes last merges the splits
  if (rc || max_splits == 1 || counters) return rc;
  launch_chained(attention_decode_bulk_combine_kernel, dim3(dim3(nq, n_seqs)), dim3(64), 0, s, part_acc, part_ml, token_of_seq, positions,
      (__nv_bfloat16*)out, out_row_stride, max_splits, nq, head_dim, split_keys);
  return check_launch("attention_decode_bulk_combine");
}
