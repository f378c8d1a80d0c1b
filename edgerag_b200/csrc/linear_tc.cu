// Weight-streaming products for the rows of a decode step on the 5th-generation tensor cores:
// out[M, N] = a[M, K] * w[N, K]^T for 1 <= M <= 64, bfloat16 operands, float accumulation.
//
// The work is reading w once at memory speed.  A block owns 128 rows of w and a slice of k:
//
//   warp 0 (copy)   one thread brings tiles of w (128 rows x 64 k, 16 KB) and of a (up to 64 rows x 64 k)
//                   into 128-byte-swizzled shared memory with TMA tensor copies, eight stages deep, so
//                   that more than a hundred kilobytes per SM are on their way at any time; the tiles of
//                   w (constants) are asked for before the wait on the kernel before this one
//   warp 1 (issue)  one thread issues tcgen05.mma with the rows of w as the M = 128 side and the rows of a
//                   as the N side (16 to 64): the accumulator is 16 to 64 columns of TMEM and costs no
//                   registers, however many rows a has
//   all four warps  afterwards read the accumulator (a thread = a row of w), hand it over through shared
//                   memory, and finish: plain store, the SwiGLU gate, or the rotary encoding with the
//                   cache write
//
// Products with few rows of w are split over k between the blocks of a cluster (up to 8, on as many
// SMs); each block then finishes a share of the rows of a, adding all blocks' sums for them in rank order
// through distributed shared memory.  The split is a function of N and K alone, and a row of `a` is a column of the
// accumulator that no other row touches: an output's bits do not depend on how many rows a has.
//
// Or the k of a tile is split over independent blocks (no cluster) that each leave their float sums as one
// of `splits` partial results [M, N], for a consumer that adds them in order while it reads (the residual
// add + norm after the attention output and the down projection).  A block of such a launch takes only
// the stages its slice of k needs, so that two fit an SM or one fits beside the kernel before it, and all
// its first tiles of w are on their way before that kernel has finished.
//
// Every wait is bounded; a thread that gives up raises a block-wide flag, the block lets its copies land,
// records 4000000 + block in *status (if given), frees its TMEM and writes nothing.
#include <stdarg.h>
#include <stdio.h>

#undef ERB_ELEM
#define ERB_ELEM 1
#include "tc_common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

constexpr int kTileN = 128;              // rows of w per block (the M side of the instruction)
constexpr int kTileK = 64;               // k per stage: one 128-byte swizzle span
constexpr int kStages = 8;
constexpr int kMaxRows = 64;             // rows of a
constexpr int kThreads = 128;
constexpr uint32_t kWBytes = kTileN * kTileK * 2;      // 16 KB
constexpr uint32_t kABytesMax = kMaxRows * kTileK * 2; // 8 KB
constexpr uint32_t kStageBytes = kWBytes + kABytesMax;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
constexpr uint32_t kTmemCols = 64;
constexpr int kMaxCluster = 8;

struct Epilogue {
  int mode;                    // 0: bfloat16 out, 1: float out, 2: gated (w rows: 64 gate + 64 up per tile), 3: rotary + cache write,
                               // 4: float partial results [splits][M][ldo], one per slice of k (no cluster)
  // mode 3
  const int* positions;        // per row of a
  const float* inv_freq;       // [head_dim / 2]
  const int* slots;            // per row of a: page * page_size + offset, negative: write no k, v
  __nv_bfloat16* k_pages;      // [page][kv head][offset][head_dim]
  __nv_bfloat16* v_pages;
  int nq, nkv, head_dim, page_size;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// MT: rows of `a` rounded up to the N side of the instruction (16, 32, 48, 64).
template <int MT>
__global__ void __launch_bounds__(kThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, void* __restrict__ out,
                 int M, int N, int K, int ldo, int splits, Epilogue ep, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kStages + 1];      // full, empty, accumulator done
  __shared__ int s_abort;
  __shared__ uint32_t tmem_slot;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]), done_bar = smem_u32(&bars[2 * kStages]);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, rank = blockIdx.y;                // (a cluster is the blocks of one tile: its ranks along y)
  const bool gated = ep.mode == 2;
  // rows of w of this tile: 128 neighbours, or for the gated product 64 gate rows and the 64 up rows that go with them
  const int n0 = tile * (gated ? kTileN / 2 : kTileN);
  const bool parts = ep.mode == 4;
  const bool clustered = splits > 1 && !parts;
  const int k_blocks = (K + kTileK - 1) / kTileK;
  const int per_rank = (k_blocks + splits - 1) / splits;
  // partial results: slices as even as they get; a cluster: whole shares, the last one short
  const int kb0 = parts ? (int)((long long)rank * k_blocks / splits) : rank * per_rank;
  const int kb1 = parts ? (int)((long long)(rank + 1) * k_blocks / splits) : min(k_blocks, kb0 + per_rank);
  const int n_kb = max(0, kb1 - kb0);

  constexpr uint32_t kABytes = MT * kTileK * 2;
  // The tiles of w are constants: the copy thread asks for the first stages as soon as it has set up the
  // barriers, before the block's other preparations and before the kernel before this one has finished.
  auto ask_w = [&](int i) {
    const int s = i % kStages;
    mbar_expect(full0 + 8 * s, kWBytes + kABytes);
    const uint32_t dst = base + s * kStageBytes;
    if (gated) {
      tma_load_2d(dst, &map_w, (kb0 + i) * kTileK, n0, full0 + 8 * s);
      tma_load_2d(dst + kWBytes / 2, &map_w, (kb0 + i) * kTileK, N + n0, full0 + 8 * s);
    } else {
      tma_load_2d(dst, &map_w, (kb0 + i) * kTileK, n0, full0 + 8 * s);
    }
  };
  const int ahead = min(kStages, n_kb);
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(done_bar, 1);
    s_abort = 0;
    mbar_init_fence();
    for (int i = 0; i < ahead; ++i) ask_w(i);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int* abort_flag = &s_abort;
  int asked = tid == 0 ? ahead : 0;     // stages the copy thread has asked for

  if (warp == 0) {
    if (lane == 0) {
      // the tiles of a (the output of the kernel before this one) only after the wait
      auto ask_a = [&](int i) {
        const int s = i % kStages;
        tma_load_2d(base + s * kStageBytes + kWBytes, &map_a, (kb0 + i) * kTileK, 0, full0 + 8 * s);
      };
      chain_wait();
      for (int i = 0; i < ahead; ++i) ask_a(i);
      asked = ahead;
      for (int i = ahead; i < n_kb; ++i) {
        if (!mbar_wait_or_abort(empty0 + 8 * (i % kStages), ((i / kStages) - 1) & 1, abort_flag)) break;
        ask_w(i);
        ask_a(i);
        asked = i + 1;
      }
    } else {
      chain_wait();
    }
  } else {
    chain_wait();
    if (warp == 1 && lane == 0) {
      constexpr uint32_t idesc = mma_idesc(kTileN, MT, false);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % kStages;
        ok = mbar_wait_or_abort(full0 + 8 * s, (i / kStages) & 1, abort_flag);
        if (!ok) break;
        fence_after_sync();
        const uint64_t dw = make_desc(base + s * kStageBytes), da = make_desc(base + s * kStageBytes + kWBytes);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) mma_bf16(tmem, dw + 2 * k, da + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        mma_commit(empty0 + 8 * s);
      }
      if (ok) mma_commit(done_bar);
    }
  }
  // ---- the accumulator: lane = row of w, column = row of a ----
  bool ok = true;
  if (n_kb > 0) {
    if (lane == 0) ok = mbar_wait_or_abort(done_bar, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok) != 0;
  }
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) {
      for (int i = max(0, asked - kStages); i < asked; ++i) mbar_wait(full0 + 8 * (i % kStages), (i / kStages) & 1);
      if (status) atomicCAS(status, 0, 4000000 + (int)blockIdx.x);
    }
    __syncthreads();
    if (clustered) { cluster_sync_all(); cluster_sync_all(); }
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    return;
  }
  // Every thread puts its row of the accumulator into shared memory as sums[m][row of w] (the stages are
  // free now), where the threads that finish a value, or the first block of the cluster, find it.
  float* sums = reinterpret_cast<float*>(smem);                 // [MT][128]
  fence_after_sync();
  {
    const uint32_t t_lane = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int c = 0; c < MT / 16; ++c) {
      float v[16];
      if (n_kb > 0) {
        tmem_ld16(t_lane + 16 * c, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) sums[(16 * c + i) * kTileN + tid] = v[i];
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  // With the k of a tile split over a cluster, every block finishes the rows m of a with m % splits == its
  // rank: it adds what all blocks hold for those rows, in rank order (its own part in its place), reading
  // the others' through distributed shared memory, 16 bytes at a time and all parts of a value at once.
  const int m_first = clustered ? rank : 0, m_step = clustered ? splits : 1;
  const int m_count = M > m_first ? (M - m_first + m_step - 1) / m_step : 0;
  if (clustered) {
    cluster_sync_all();
    uint32_t remote[kMaxCluster];
#pragma unroll
    for (int o = 0; o < kMaxCluster; ++o)
      asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[o]) : "r"(smem_u32(sums)), "r"(o < splits ? o : 0));
    for (int idx = tid; idx < m_count * (kTileN / 4); idx += kThreads) {
      const int m = m_first + (idx / (kTileN / 4)) * m_step, c4 = idx % (kTileN / 4);
      const uint32_t off = (uint32_t)(m * kTileN + c4 * 4) * 4u;
      float4 part[kMaxCluster];
#pragma unroll
      for (int o = 0; o < kMaxCluster; ++o) {
        part[o] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (o < splits)
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(part[o].x), "=f"(part[o].y), "=f"(part[o].z), "=f"(part[o].w) : "r"(remote[o] + off));
      }
      float4 total = part[0];
#pragma unroll
      for (int o = 1; o < kMaxCluster; ++o) {
        if (o < splits) { total.x += part[o].x; total.y += part[o].y; total.z += part[o].z; total.w += part[o].w; }
      }
      *reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(sums) + off) = total;
    }
    cluster_sync_all();                // (every block's shared memory had to stay until all had read it)
    __syncthreads();
  }

  // ---- finishing ----
  if (parts) {
    // 16 bytes a thread, a row of a after the other (scattered 4-byte stores straight from the accumulator's
    // registers were slower: 10.6 against 9.6 us for the down projection at 64 rows)
    float* dst = reinterpret_cast<float*>(out) + (size_t)rank * M * ldo;
    for (int idx = tid; idx < M * (kTileN / 4); idx += kThreads) {
      const int m = idx / (kTileN / 4), c4 = (idx % (kTileN / 4)) * 4, n = n0 + c4;
      const float4 v = *reinterpret_cast<const float4*>(sums + m * kTileN + c4);
      if (n + 3 < N) {
        *reinterpret_cast<float4*>(dst + (size_t)m * ldo + n) = v;
      } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
        for (int j = 0; j < 4 && n + j < N; ++j) dst[(size_t)m * ldo + n + j] = e[j];
      }
    }
  } else if (ep.mode <= 1) {
    for (int idx = tid; idx < m_count * kTileN; idx += kThreads) {
      const int m = m_first + (idx / kTileN) * m_step, n = n0 + idx % kTileN;
      if (n >= N) continue;
      const float v = sums[m * kTileN + idx % kTileN];
      if (ep.mode == 1) reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
      else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
    }
  } else if (ep.mode == 2) {
    // silu(g) * u, both rounded to bfloat16 first (as if the product had been stored)
    for (int idx = tid; idx < m_count * (kTileN / 2); idx += kThreads) {
      const int m = m_first + (idx / (kTileN / 2)) * m_step, e = idx % (kTileN / 2), n = n0 + e;
      if (n >= N) continue;
      const float g = __bfloat162float(__float2bfloat16_rn(sums[m * kTileN + e]));
      const float u = __bfloat162float(__float2bfloat16_rn(sums[m * kTileN + kTileN / 2 + e]));
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(silu_mul(g, u));
    }
  } else {
    // rotary halves on q and k heads (a thread takes a pair), cache write of k and v
    const int D = ep.head_dim, half = D / 2;
    const int heads_per_tile = kTileN / D;
    for (int idx = tid; idx < m_count * (kTileN / 2); idx += kThreads) {
      const int m = m_first + (idx / (kTileN / 2)) * m_step, pair = idx % (kTileN / 2);
      const int head_local = pair / half, e = pair % half;
      const int head = tile * heads_per_tile + head_local;
      if (head >= ep.nq + 2 * ep.nkv) continue;
      const float* row = sums + m * kTileN + head_local * D;
      const float lo = __bfloat162float(__float2bfloat16_rn(row[e]));
      const float hi = __bfloat162float(__float2bfloat16_rn(row[e + half]));
      const int slot = ep.slots[m];
      const size_t page = slot >= 0 ? slot / ep.page_size : 0, off = slot >= 0 ? slot % ep.page_size : 0;
      if (head < ep.nq + ep.nkv) {
        float sn, cs, o0, o1;
        sincosf((float)ep.positions[m] * ep.inv_freq[e], &sn, &cs);
        rotate_pair(lo, hi, cs, sn, o0, o1);
        __nv_bfloat16* dst = nullptr;
        if (head < ep.nq) dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + (size_t)head * D;
        else if (slot >= 0) dst = ep.k_pages + ((page * ep.nkv + (head - ep.nq)) * ep.page_size + off) * D;
        if (dst) { dst[e] = __float2bfloat16_rn(o0); dst[e + half] = __float2bfloat16_rn(o1); }
      } else if (slot >= 0) {
        __nv_bfloat16* dst = ep.v_pages + ((page * ep.nkv + (head - ep.nq - ep.nkv)) * ep.page_size + off) * D;
        dst[e] = __float2bfloat16_rn(lo);
        dst[e + half] = __float2bfloat16_rn(hi);
      }
    }
  }
}

// A tensor map over rows of 64-k boxes: matrix[rows][K] with row stride ld, boxes of box_rows rows.
int matrix_map(CUtensorMap* out, const void* p, int rows, int K, int ld, int box_rows) {
  static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  const auto key = std::make_tuple(p, rows, K, ld, box_rows);
  auto it = maps.find(key);
  if (it == maps.end()) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, elem,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ERB_ERR_CUDA, "linear_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (maps.size() > 8192) maps.clear();
    it = maps.emplace(key, m).first;
  }
  *out = it->second;
  return ERB_OK;
}

int* g_status_word = nullptr;

// Blocks that share a tile of w rows (each takes a slice of k): as many as make about one block per SM,
// at most 8, and no more than there are stages of 64 k.  A function of N and K only.
int k_splits(int n_tiles, int K) {
  const int k_blocks = (K + kTileK - 1) / kTileK;
  int s = sm_count() / n_tiles;
  if (s > kMaxCluster) s = kMaxCluster;
  while (s > 1 && k_blocks / s < 2) --s;
  return s < 1 ? 1 : s;
}

// Independent blocks per tile of w rows for partial results: as many as make about one block per SM, each
// with at least two stages of 64 k, at most kMaxParts.  A function of N and K only.
constexpr int kMaxParts = 16;
int k_parts(int n_tiles, int K) {
  const int k_blocks = (K + kTileK - 1) / kTileK;
  int s = sm_count() / n_tiles;
  if (s > kMaxParts) s = kMaxParts;
  while (s > 1 && k_blocks / s < 2) --s;
  return s < 1 ? 1 : s;
}

template <int MT>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K, int ldo, int n_tiles, int splits,
           const Epilogue& ep, cudaStream_t stream) {
  auto kern = linear_tc_kernel<MT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "linear_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, splits);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  if (ep.mode == 4) {
    // the stages that the longest slice of k touches, and room for the sums [MT][128] afterwards
    const int k_blocks = (K + kTileK - 1) / kTileK, longest = (k_blocks + splits - 1) / splits;
    const uint32_t stages = (uint32_t)(longest < kStages ? longest : kStages);
    const uint32_t need = stages * kStageBytes, sums = (uint32_t)MT * kTileN * 4;
    cfg.dynamicSmemBytes = (need > sums ? need : sums) + 1024;
  }
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (splits > 1 && ep.mode != 4) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = splits;
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
  cudaLaunchKernelEx(&cfg, kern, mw, ma, out, M, N, K, ldo, splits, ep, g_status_word);
  return check_launch("linear_tc");
}

int run(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldo, int w_rows, const Epilogue& ep,
        cudaStream_t stream) {
  if (M <= 0) return ERB_OK;
  if (M > kMaxRows) return fail(ERB_ERR_UNSUPPORTED, "linear_tc: %d rows (at most %d)", M, kMaxRows);
  if (N <= 0 || K <= 0 || lda < K || ldw < K) return fail(ERB_ERR_ARG, "linear_tc: bad sizes");
  if ((K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return fail(ERB_ERR_UNSUPPORTED, "linear_tc: K and the leading dimensions must be multiples of 8, operands 16-byte aligned");
  const int MT = (M + 15) / 16 * 16;
  CUtensorMap mw, ma;
  int rc;
  if ((rc = matrix_map(&mw, w, w_rows, K, ldw, ep.mode == 2 ? kTileN / 2 : kTileN)) || (rc = matrix_map(&ma, a, M, K, lda, MT))) return rc;
  const int per_tile = ep.mode == 2 ? kTileN / 2 : kTileN;
  const int n_tiles = ((ep.mode == 3 ? w_rows : N) + per_tile - 1) / per_tile;
  const int splits = ep.mode == 4 ? k_parts(n_tiles, K) : k_splits(n_tiles, K);
  switch (MT) {
    case 16: return launch<16>(mw, ma, out, M, N, K, ldo, n_tiles, splits, ep, stream);
    case 32: return launch<32>(mw, ma, out, M, N, K, ldo, n_tiles, splits, ep, stream);
    case 48: return launch<48>(mw, ma, out, M, N, K, ldo, n_tiles, splits, ep, stream);
    default: return launch<64>(mw, ma, out, M, N, K, ldo, n_tiles, splits, ep, stream);
  }
}

}  // namespace

// The device word (int) to which the kernels report a wait that ran out (code 4000000 + block); null:
// nowhere.  Kept until set again.
ERB_EXPORT int erb_linear_tc_set_status_word(int* status) {
  g_status_word = status;
  return ERB_OK;
}

// out[M, N] = a[M, K] * w[N, K]^T for 1 <= M <= 64; out is bfloat16, or float with out_f32.
ERB_EXPORT int erb_linear_tc(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldo,
                             int out_f32, void* stream) {
  if (ldo < N) return fail(ERB_ERR_ARG, "linear_tc: bad sizes");
  Epilogue ep = {};
  ep.mode = out_f32 ? 1 : 0;
  return run(a, w, out, M, N, K, lda, ldw, ldo, N, ep, (cudaStream_t)stream);
}

// The number of partial results that erb_linear_tc_parts leaves for a product with N rows of w and K columns.
ERB_EXPORT int erb_linear_tc_parts_count(int N, int K) { return k_parts((N + kTileN - 1) / kTileN, K); }

// parts[s][M][ldo] (float), s < erb_linear_tc_parts_count(N, K): the sums over the s-th slice of k of
// a[M, K] * w[N, K]^T; the product is their sum.  1 <= M <= 64.
ERB_EXPORT int erb_linear_tc_parts(const void* a, const void* w, void* parts, int M, int N, int K, int lda, int ldw, int ldo,
                                   void* stream) {
  if (ldo < N || (ldo & 3) || ((uintptr_t)parts & 15)) return fail(ERB_ERR_ARG, "linear_tc_parts: bad sizes");
  Epilogue ep = {};
  ep.mode = 4;
  return run(a, w, parts, M, N, K, lda, ldw, ldo, N, ep, (cudaStream_t)stream);
}

// Gated product: w holds N gate rows and then N up rows ([2N, K]); out[M, N] = silu(g) * u with
// g = a * gate^T and u = a * up^T, each rounded to bfloat16 before the gate.
ERB_EXPORT int erb_linear_tc_glu(const void* a, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldo,
                                 void* stream) {
  if (ldo < N) return fail(ERB_ERR_ARG, "linear_tc_glu: bad sizes");
  Epilogue ep = {};
  ep.mode = 2;
  return run(a, w, out, M, N, K, lda, ldw, ldo, 2 * N, ep, (cudaStream_t)stream);
}

// The attention input projection with the rotary encoding and the cache write in its epilogue:
// w = [Wq; Wk; Wv] of shape [(nq + 2 nkv) * head_dim, K]; q is rotated and written to
// out[M, >= nq * head_dim], k is rotated and, with v, written to each token's cache slot.  The products
// are rounded to bfloat16 before the rotation.  head_dim 32, 64 or 128 (a tile of 128 rows of w holds
// whole heads), full rotation.
ERB_EXPORT int erb_linear_tc_rope_supported(int head_dim) { return head_dim == 32 || head_dim == 64 || head_dim == 128; }

ERB_EXPORT int erb_linear_tc_rope(const void* a, const void* w, void* out, int M, int K, int lda, int ldw, int ldo, int nq,
                                  int nkv, int head_dim, const int* positions, const float* inv_freq, const int* slots,
                                  void* k_pages, void* v_pages, int page_size, void* stream) {
  if (!erb_linear_tc_rope_supported(head_dim))
    return fail(ERB_ERR_UNSUPPORTED, "linear_tc_rope: head_dim %d (takes 32, 64, 128)", head_dim);
  if (nq <= 0 || nkv <= 0 || page_size <= 0 || !positions || !inv_freq || !slots || !k_pages || !v_pages || ldo < nq * head_dim)
    return fail(ERB_ERR_ARG, "linear_tc_rope: bad arguments");
  Epilogue ep = {3, positions, inv_freq, slots, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, nq, nkv, head_dim, page_size};
  const int rows = (nq + 2 * nkv) * head_dim;
  return run(a, w, out, M, rows, K, lda, ldw, ldo, rows, ep, (cudaStream_t)stream);
}
