// Causal attention for portions of prompts on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// bfloat16, head size 64, queries of one (sequence, query head) in tiles of 128 rows, keys and
// values read straight from cache pages in tiles of 128 keys.
//
//   S = Q K^T      tcgen05.mma  M=128 N=64 K=16 x4    A = Q tile, B = K tile, both K-major in
//                  shared memory (rows of 128 bytes, 128-byte swizzle), accumulator in TMEM
//   softmax        two threads per query row, 32 score columns each: tcgen05.ld of their part of the
//                  S row, reference max / denominator in float, P rounded to bfloat16 into shared memory
//   O += P V       tcgen05.mma  M=128 N=64 K=16 x4    A = P (K-major), B = V tile as stored in the
//                  cache (rows = keys, 64 contiguous values: the MN-major operand form); O stays in TMEM
//
// K and V tiles of 64 keys are brought in with cp.async 16-byte copies (zero-filled past the last
// visible key), two tiles ahead, four stages.  One block is 256 threads and 113 KB of shared
// memory, so two blocks (16 warps) share an SM; each allocates 256 TMEM columns.
//
// Every wait on an mbarrier is bounded: on a timeout the block records an error in *status,
// skips the rest of its work, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <tuple>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#undef ERB_ELEM
#define ERB_ELEM 1
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

constexpr int BM = 128;       // query rows per block
constexpr int BN = 64;        // keys per tile
constexpr int HD = 64;        // head size
constexpr int kThreads = 256;     // two threads per query row
constexpr int kKvStages = 4;      // K and V tiles in shared memory
constexpr uint32_t kQBytes = BM * HD * 2;           // 16 KB: the Q tile
constexpr uint32_t kTileBytes = BN * HD * 2;        // 8 KB: one K or V tile
constexpr uint32_t kPBytes = BM * BN * 2;           // 16 KB: one P tile (two of them)
// 114,752 bytes of tiles + 64 of barriers: two blocks fit in an SM's 227 KB (each block also costs 1 KB of
// system shared memory), which needs the dynamic shared memory to start 1024-byte aligned: checked at run time.
constexpr uint32_t kSmemBytes = kQBytes + 2 * kKvStages * kTileBytes + 2 * kPBytes + 64;
constexpr uint32_t kTmemCols = 256;                 // S(even tiles): columns 0..63, S(odd): 64..127, O: 128..191
constexpr uint32_t kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` in a tile of 128-byte rows with the
// 128-byte swizzle: groups of 8 rows take 1024 bytes, the chunk index is XORed with the row.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// Shared-memory matrix descriptor: 128-byte swizzle, 1024 bytes between groups of 8 rows.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                           // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                           // layout: 128-byte swizzle
  return d;
}

// Instruction descriptors: float accumulate, bfloat16 operands, M = 128.
constexpr uint32_t kIdescS = (1u << 4) | (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);
constexpr uint32_t kIdescO = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /*B is MN-major*/ |
                             ((HD >> 3) << 17) | ((BM >> 4) << 24);

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Waits for the phase with the given parity; gives up after kSpinLimit polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {          // 2^x, one instruction; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Pipeline (one block, tile j of 64 keys):
//   copies for tile j+2 are in flight (cp.async, four stages);
//   S(j+1) = Q K(j+1)^T is issued before the softmax of tile j, into the other half of the S columns;
//   the softmax of tile j reads S(j) from TMEM, writes P(j) (bfloat16) to one of two shared buffers;
//   O += P(j) V(j) accumulates in TMEM and is only waited for when its inputs are reused two tiles
//   later, or when the running maximum of a row grew by more than 2^8 and O must be rescaled.
// The softmax keeps a reference maximum per row that only moves in such jumps (p <= 2^8 in between), so
// the O rescale, the one step that would serialise the tensor core behind the CUDA cores, is rare.
__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride,
                            const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                            const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_starts,
                            const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, int out_row_stride,
                            int n_seqs, int nq, int nkv, int page_size, float scale_log2, int* __restrict__ status) {
  chain_wait();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {                       // the swizzled tiles need 1024-byte aligned bases
    if (threadIdx.x == 0) atomicCAS(status, 0, 3000000);
    return;
  }
  uint8_t* smem = smem_raw;
  const uint32_t sQ = base, sK0 = base + kQBytes, sV0 = sK0 + kKvStages * kTileBytes, sP0 = sV0 + kKvStages * kTileBytes;
  const uint32_t bar0 = sP0 + 2 * kPBytes;          // bar_s[0], bar_s[1], bar_pv[0], bar_pv[1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar0 - base) + 32);

  // Two threads per query row: thread (row, half) owns score columns half*32 .. +31 of a tile and
  // output columns half*32 .. +31.  A warp reaches the 32 TMEM lanes of its quarter.
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & (BM - 1), half = tid >> 7;
  const int h = blockIdx.y;
  const int kvh = h / (nq / nkv);

  // Which sequence and which 128-row tile of it this block owns.  Blocks are numbered from the last
  // tile backwards: later tiles of a prompt see more keys and take longer, so they should start first.
  int tile = (int)(gridDim.x - 1 - blockIdx.x), seq = -1, q0 = 0, rows = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const int begin = seq_starts[s], len = seq_starts[s + 1] - begin;
    const int n_tiles = (len + BM - 1) / BM;
    if (tile < n_tiles) { seq = s; q0 = begin + tile * BM; rows = min(BM, len - tile * BM); break; }
    tile -= n_tiles;
  }
  if (seq < 0) return;  // the grid was sized with an upper bound
  if (*reinterpret_cast<volatile int*>(status) != 0) return;  // an earlier block gave up: do not pile on
  const int pos0 = positions[q0];
  const int last_key = pos0 + rows - 1;
  const int n_kv = last_key / BN + 1;
  const int* bt = block_tables + (size_t)seq * max_pages;

  if (tid == 0) {
#pragma unroll
    for (int b = 0; b < 4; ++b) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8 * b));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // Each thread copies chunk (tid % 8) of rows (tid / 8) + 32 i, so a warp covers whole 128-byte rows.
  const int lc = tid & 7, lr = tid >> 3;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  auto load_kv = [&](int j) {               // always commits a group, empty past the last tile
    if (j < n_kv) {
      const int stage = j % kKvStages;
      const uint32_t dK = sK0 + stage * kTileBytes, dV = sV0 + stage * kTileBytes;
#pragma unroll
      for (int i = 0; i < BN / 32; ++i) {
        const int r = lr + 32 * i;
        const int key = j * BN + r;
        const bool valid = key <= last_key;
        size_t off = 0;
        if (valid) {
          const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
          const int po = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
          off = (((size_t)bt[pi] * nkv + kvh) * page_size + po) * HD + lc * 8;
        }
        cp_async16(dK + swz(r, lc), k_pages + off, valid);
        cp_async16(dV + swz(r, lc), v_pages + off, valid);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < BM / 32; ++i) {
    const int r = lr + 32 * i;
    const bool valid = r < rows;
    const __nv_bfloat16* src = q + (size_t)(q0 + (valid ? r : 0)) * q_row_stride + (size_t)h * HD + lc * 8;
    cp_async16(sQ + swz(r, lc), src, valid);
  }
  load_kv(0);
  load_kv(1);
  cp_async_wait<1>();                       // Q and tile 0 have landed
  fence_async_proxy();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes of TMEM
  const uint32_t t_o = t_lane + 2 * BN + half * 32;                      // this thread's 32 output columns
  const int my_pos = pos0 + row;
  const uint64_t dq = make_desc(sQ);
  bool ok = true;

  auto issue_s = [&](int j) {               // thread 0: S(j) into S columns (j & 1) * 64
    const uint64_t dk = make_desc(sK0 + (j % kKvStages) * kTileBytes);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) mma_bf16(tmem + (j & 1) * BN, dq + 2 * k, dk + 2 * k, kIdescS, k > 0);
    mma_commit(bar0 + 8 * (j & 1));
  };
  if (tid == 0) issue_s(0);

  float m_ref = -INFINITY, l_run = 0.f;     // l_run: this thread's half of the row's denominator
  for (int j = 0; j < n_kv; ++j) {
    // (A) tile j+1 is in shared memory for everyone; everyone is done with iteration j-1
    cp_async_wait<0>();
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (tid == 0 && ok && j + 1 < n_kv) issue_s(j + 1);
    // the stage tile j+2 goes into was last read by P V of tile j-2
    if (ok && j >= 2 && !mbar_wait(bar0 + 16 + 8 * (j & 1), ((j - 2) >> 1) & 1)) ok = false;
    load_kv(j + 2);

    if (ok && !mbar_wait(bar0 + 8 * (j & 1), (j >> 1) & 1)) ok = false;
    fence_after_sync();
    float s[32];
    if (ok) {
      tmem_ld32(t_lane + (j & 1) * BN + half * 32, s);
      tmem_ld_wait();
    }
    const int key0 = j * BN + half * 32;
    float m_half = -INFINITY;
    if (key0 + 31 <= my_pos) {              // every key of this half is visible to this row
#pragma unroll
      for (int i = 0; i < 32; ++i) m_half = fmaxf(m_half, s[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (key0 + i > my_pos) s[i] = -INFINITY;
        m_half = fmaxf(m_half, s[i]);
      }
    }
    m_half *= scale_log2;                   // scale > 0: the maximum of the scaled scores
    // The two threads of a row exchange their maxima through the P buffer of this tile, which is free
    // (P V of tile j-2 was waited for above): each writes into the first bytes of its partner's part of
    // the row and reads its own part, which nobody else touches until the thread overwrites it with P.
    uint8_t* p_row = smem + (sP0 - base) + (j & 1) * kPBytes;
    *reinterpret_cast<float*>(p_row + swz(row, (half ^ 1) * 4)) = m_half;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");   // only the two warps that share these rows
    const float m_tile = fmaxf(m_half, *reinterpret_cast<const float*>(p_row + swz(row, half * 4)));
    // The reference maximum moves only when the row's maximum grew by more than 2^8.
    float alpha = 1.f;
    const bool jump = m_tile > m_ref + 8.f;               // true on the first tile (m_ref = -inf)
    if (jump) {
      alpha = fast_exp2(m_ref - m_tile);                  // 0 on the first tile
      m_ref = m_tile;
    }
    if (j > 0 && __any_sync(0xffffffffu, jump)) {
      // O of this warp's rows is rescaled in TMEM; P V of tile j-1 must have landed first
      if (ok && !mbar_wait(bar0 + 16 + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1)) ok = false;
      fence_after_sync();
      if (ok) {
        float acc[32];
        tmem_ld32(t_o, acc);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] *= alpha;
        tmem_st32(t_o, acc);
        tmem_st_wait();
      }
    }
    float l_tile = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {           // this thread's four 16-byte chunks of the row of P
      uint32_t packed[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float p0 = fast_exp2(fmaf(s[8 * g + 2 * i], scale_log2, -m_ref));
        const float p1 = fast_exp2(fmaf(s[8 * g + 2 * i + 1], scale_log2, -m_ref));
        l_tile += p0 + p1;
        __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
        packed[i] = *reinterpret_cast<uint32_t*>(&b);
      }
      if (ok) *reinterpret_cast<uint4*>(p_row + swz(row, half * 4 + g)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    l_run = l_run * alpha + l_tile;
    fence_async_proxy();
    fence_before_sync();
    __syncthreads();                        // (B) P(j) is written, O is rescaled, S(j) has been read
    if (tid == 0 && ok) {
      fence_after_sync();
      const uint64_t dp = make_desc(sP0 + (j & 1) * kPBytes), dv = make_desc(sV0 + (j % kKvStages) * kTileBytes);
#pragma unroll
      for (int k = 0; k < BN / 16; ++k)
        mma_bf16(tmem + 2 * BN, dp + 2 * k, dv + (uint64_t)(k * (2048 >> 4)), kIdescO, (j > 0 || k > 0) ? 1u : 0u);
      mma_commit(bar0 + 16 + 8 * (j & 1));
    }
  }
  cp_async_wait<0>();
  // every P V has landed once the last two have
  if (ok && n_kv >= 2 && !mbar_wait(bar0 + 16 + 8 * ((n_kv - 2) & 1), ((n_kv - 2) >> 1) & 1)) ok = false;
  if (ok && !mbar_wait(bar0 + 16 + 8 * ((n_kv - 1) & 1), ((n_kv - 1) >> 1) & 1)) ok = false;
  fence_after_sync();
  // exchange the two halves of the denominator (through P buffer 0: no P V reads it any more)
  uint8_t* p_row = smem + (sP0 - base);
  *reinterpret_cast<float*>(p_row + swz(row, (half ^ 1) * 4)) = l_run;
  __syncthreads();
  const float l_row = l_run + *reinterpret_cast<const float*>(p_row + swz(row, half * 4));

  if (!ok) {
    atomicCAS(status, 0, 1000000 + (int)blockIdx.x);
  } else {
    float acc[32];
    tmem_ld32(t_o, acc);
    tmem_ld_wait();
    if (row < rows) {
      const float inv = 1.f / l_row;
      __nv_bfloat16* dst = out + (size_t)(q0 + row) * out_row_stride + (size_t)h * HD + half * (HD / 2);
#pragma unroll
      for (int d = 0; d < HD / 2; d += 8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 b = __floats2bfloat162_rn(acc[d + 2 * i] * inv, acc[d + 2 * i + 1] * inv);
          w[i] = *reinterpret_cast<uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(dst + d) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

// Portions of prompts only (bfloat16, head_dim 64, no window).  q / out: row t is token t of the
// batch; seq_starts: int32 [n_seqs + 1] token offsets of the sequences to process (consecutive
// rows of block_tables); n_tiles: sum over them of ceil(length / 128) (an upper bound is fine).
// status: device int, set non-zero if a block gave up waiting on the tensor cores.
ERB_EXPORT int erb_attention_prefill_tc(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                        const int* block_tables, int max_pages, const int* seq_starts,
                                        const int* positions, void* out, int out_row_stride, int n_seqs,
                                        int n_tiles, int nq, int nkv, int head_dim, int page_size, float scale,
                                        int* status, void* stream) {
  if (n_seqs <= 0 || n_tiles <= 0) return ERB_OK;
  if (head_dim != HD) return fail(ERB_ERR_UNSUPPORTED, "attention_prefill_tc: head_dim %d (this kernel takes 64)", head_dim);
  if (nq <= 0 || nkv <= 0 || nq % nkv || nq > 65535) return fail(ERB_ERR_ARG, "attention_prefill_tc: bad head counts");
  if (page_size <= 0 || max_pages <= 0 || !status) return fail(ERB_ERR_ARG, "attention_prefill_tc: bad cache arguments");
  if (q_row_stride % 8 || out_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
    return fail(ERB_ERR_UNSUPPORTED, "attention_prefill_tc: rows must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_prefill_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_chained(attention_prefill_tc_kernel, dim3(dim3(n_tiles, nq)), dim3(kThreads), kSmemBytes, (cudaStream_t)stream, 
      (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
      block_tables, max_pages, seq_starts, positions, (__nv_bfloat16*)out, out_row_stride, n_seqs, nq, nkv,
      page_size, scale_log2, status);
  return check_launch("attention_prefill_tc");
}

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
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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

template <int D, int R>   // head size; query heads per kv head (1..kMaxGroup)
__global__ void __launch_bounds__(kDecThreads)
attention_decode_bulk_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride,
                             const __nv_bfloat16* __restrict__ k_pages, const __nv_bfloat16* __restrict__ v_pages,
                             const int* __restrict__ block_tables, int max_pages,
                             const int* __restrict__ token_of_seq, const int* __restrict__ positions,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, int max_splits, int nq,
                             int nkv, int page_size, int split_keys, float scale_log2, int hg,
                             __nv_bfloat16* __restrict__ out, int out_row_stride, int* __restrict__ status) {
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
}

// Merges the splits of each (sequence, head).  The partial maxima are in the log2 domain.  The
// weights of the splits are computed by the first lanes in parallel; every output element is then
// a sum over the splits in their order.
constexpr int kCombineMaxSplits = 64;
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
int decode_head_group(int nkv, int head_dim, int page_size, int split_keys) {
  const int stage_rows = kDecWarps * (32 / (head_dim / 8)) * kKeysPerGroup;
  auto fits = [&](int hg) { return hg <= kDecWarps && (stage_rows / hg) % page_size == 0 && stage_rows / hg >= page_size; };
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
                       int split_keys, float scale_log2, void* out, int out_row_stride, int* status, cudaStream_t s) {
  const int hg = decode_head_group(nkv, D, page_size, split_keys);
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
      part_acc, part_ml, max_splits, nq, nkv, page_size, split_keys, scale_log2, hg, (__nv_bfloat16*)out, out_row_stride, status);
  return check_launch("attention_decode_bulk");
}

template <int D>
int dispatch_group(int r, const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                   const int* block_tables, int max_pages, const int* token_of_seq, const int* positions,
                   float* part_acc, float* part_ml, int max_splits, int n_seqs, int nq, int nkv, int page_size,
                   int split_keys, float scale_log2, void* out, int out_row_stride, int* status, cudaStream_t s) {
#define ERB_R(RR)                                                                                              \
  case RR: return launch_decode_bulk<D, RR>(q, q_row_stride, k_pages, v_pages, block_tables, max_pages,        \
                                            token_of_seq, positions, part_acc, part_ml, max_splits, n_seqs, nq, \
                                            nkv, page_size, split_keys, scale_log2, out, out_row_stride,       \
                                            status, s);
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

__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(bar) : "memory");
}
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
                            __nv_bfloat16* __restrict__ out, int out_row_stride, int* __restrict__ status) {
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
}

// Tensor maps over a page pool [rows = pages * kv heads * page_size][64] with boxes of `box_rows`
// rows, 128-byte swizzle.  Encoding is a host-side computation; the maps are kept per (pool, box).
std::map<std::tuple<const void*, unsigned long long, unsigned>, CUtensorMap> g_maps;
std::mutex g_maps_mutex;

int pool_map(CUtensorMap* out, const void* pool, unsigned long long rows, unsigned box_rows) {
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  const auto key = std::make_tuple(pool, rows, box_rows);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    const cuuint64_t dims[2] = {64, rows};
    const cuuint64_t strides[1] = {128};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = cuTensorMapEncodeTiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides,
                                              box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ERB_ERR_CUDA, "attention_decode_gqa: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return ERB_OK;
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
                                        void* stream) {
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
  if ((rc = pool_map(&mk, k_pages, rows, (unsigned)(hg * page_size))) || (rc = pool_map(&mv, v_pages, rows, (unsigned)(hg * page_size))) ||
      (rc = pool_map(&mkl, k_pages, rows, (unsigned)(last * page_size))) || (rc = pool_map(&mvl, v_pages, rows, (unsigned)(last * page_size))))
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
                 status);
  if ((rc = check_launch("attention_decode_gqa")) || max_splits == 1) return rc;      // a single split wrote the result itself
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

// Same contract as the general decode entry point (scratch provided by the caller, splits at
// absolute multiples of split_keys), for bfloat16 with head_dim 32 / 64 / 128, no window, at most
// 8 query heads per kv head, and page rows that are 16-byte multiples.
ERB_EXPORT int erb_attention_decode_bulk(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                         const int* block_tables, int max_pages, const int* token_of_seq,
                                         const int* positions, void* out, int out_row_stride, float* part_acc,
                                         float* part_ml, int max_splits, int n_seqs, int nq, int nkv, int head_dim,
                                         int page_size, int split_keys, float scale, int* status, void* stream) {
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
                                     scale_log2, out, out_row_stride, status, s); break;
    case 64: rc = dispatch_group<64>(r, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                                     positions, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size, split_keys,
                                     scale_log2, out, out_row_stride, status, s); break;
    case 128: rc = dispatch_group<128>(r, q, q_row_stride, k_pages, v_pages, block_tables, max_pages, token_of_seq,
                                       positions, part_acc, part_ml, max_splits, n_seqs, nq, nkv, page_size,
                                       split_keys, scale_log2, out, out_row_stride, status, s); break;
    default: return fail(ERB_ERR_UNSUPPORTED, "attention_decode_bulk: head_dim %d (takes 32, 64, 128)", head_dim);
  }
  if (rc || max_splits == 1) return rc;      // a single split wrote the result itself
  launch_chained(attention_decode_bulk_combine_kernel, dim3(dim3(nq, n_seqs)), dim3(64), 0, s, part_acc, part_ml, token_of_seq, positions,
      (__nv_bfloat16*)out, out_row_stride, max_splits, nq, head_dim, split_keys);
  return check_launch("attention_decode_bulk_combine");
}
