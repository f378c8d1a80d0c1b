// Causal attention for portions of prompts on the 5th-generation tensor cores (tcgen05 + TMEM),
// with the block's warps specialised by role.
//
// bfloat16, head size 64, cache pages of 8, 16, 32, 64 or 128 tokens.  A block owns 256 query rows
// of one (sequence, query head) as two tiles of 128 rows, A and B, and walks the keys in tiles of
// 128.  Both query tiles use the same key and value tiles, so every byte of K and V that reaches
// shared memory serves 256 rows.
//
//   warp 17 (copy)    brings K(j) and V(j) from the cache pages into 128-byte-swizzled shared memory
//                     with TMA tensor copies, one copy per page, up to four tiles of each in flight
//   warp 16 (issue)   one thread issues S_t(j) = Q_t K(j)^T (M 128, N 128, K 64) and
//                     O_t += P_t(j) V(j) (M 128, N 64, K 128) for t = A, B; accumulators in TMEM
//   warps 0-7, 8-15   softmax of tile A and of tile B: two threads per query row, each with 64 of the
//                     tile's 128 keys; a thread reads its scores from TMEM 32 at a time, exponentiates
//                     them, and writes P rounded to bfloat16 back to TMEM, from where the second product
//                     reads it as its A operand (P never passes through shared memory)
//
// The two softmax groups work on alternate products: while group A exponentiates S_A(j), the tensor
// core computes S_B(j) and O_A += P_A(j-1) V(j-1).  Nobody but the copy warp touches addresses of
// pages, and no block-wide barrier is taken inside the loop: every hand-over is an mbarrier
// (K/V tile full, tile free again, S ready, P ready, product done).
//
// A row's reference maximum is set on the first tile and then only moves when a tile's sum of P shows
// that it has become far too low (P is a floating-point number: a reference that is low by twenty powers
// of two costs no precision).  So most tiles need no search for a maximum and no rescaling of O.
//
// A portion that is short against its past (512 new tokens after 7,000 cached ones) gives few blocks,
// each with a long walk over the keys.  The launch may then cut every block's key tiles into
// `key_splits` ranges, one block per range (blockIdx.z): a block leaves its rows' unnormalised O, reference
// maximum and sum in scratch, and a second kernel merges the ranges of each row.
//
// Every wait is bounded: a thread that gives up raises a block-wide flag, every other wait of the
// block then ends too, the block records a code in *status, lets its copies land, frees its TMEM
// and returns.
#include <stdarg.h>
#include <stdio.h>

#undef ERB_ELEM
#define ERB_ELEM 1
#include "tc_common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

constexpr int BM = 128;               // rows of a query tile
constexpr int BN = 128;               // keys of a key/value tile
constexpr int HD = 64;                // head size
constexpr int kRowsPerBlock = 2 * BM;
constexpr int kKStages = 4, kVStages = 4;   // key and value tiles in shared memory (powers of two)
constexpr int kSoftmaxWarps = 16;           // per query tile 8 warps: two threads per row, 64 keys of a tile each
constexpr int kGroupThreads = 2 * BM;       // threads of one softmax group
constexpr int kIssueWarp = kSoftmaxWarps, kCopyWarp = kSoftmaxWarps + 1;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr uint32_t kQBytes = BM * HD * 2;               // 16 KB per query tile
constexpr uint32_t kKvBytes = BN * HD * 2;              // 16 KB per key or value tile
// barriers, in this order (8 bytes each)
constexpr int kBarKFull = 0, kBarKEmpty = kBarKFull + kKStages, kBarVFull = kBarKEmpty + kKStages,
              kBarVEmpty = kBarVFull + kVStages, kBarSFull = kBarVEmpty + kVStages, kBarPFull = kBarSFull + 2,
              kBarPvDone = kBarPFull + 2, kNumBars = kBarPvDone + 2;
constexpr uint32_t kSmemTiles = 2 * kQBytes + kKStages * kKvBytes + kVStages * kKvBytes;
constexpr uint32_t kSmemExchange = 2 * 2 * BM * 2 * 4;  // two floats (maximum, sum) per (group, row, half of the row)
constexpr uint32_t kSmemBytes = kSmemTiles + kSmemExchange + 8 * kNumBars + 16 + 1024;   // + abort flag, TMEM slot, alignment slack
// TMEM columns: S_A 0..127, S_B 128..255, O_A 256..319, O_B 320..383, P_A 384..447, P_B 448..511
// (P: two bfloat16 per 32-bit column, the row's keys in order: the A operand of the second product)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;
constexpr float kSumLimit = 1048576.f;   // a tile's sum of P from which on the reference maximum is moved (2^20)
constexpr uint32_t kIdescS = mma_idesc(BM, BN, false);
constexpr uint32_t kIdescO = mma_idesc(BM, HD, true);

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __nv_bfloat16* __restrict__ q, int q_row_stride,
                         const int* __restrict__ block_tables, int max_pages, const int* __restrict__ seq_starts,
                         const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, int out_row_stride,
                         int n_seqs, int nq, int nkv, int page_size, float scale_log2, int* __restrict__ status,
                         int key_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;             // the swizzle repeats every 1024 bytes
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sQ = base, sK = sQ + 2 * kQBytes, sV = sK + kKStages * kKvBytes;
  float* exchange = reinterpret_cast<float*>(smem + kSmemTiles);                     // [group][row][half]
  const uint32_t bars = sV + kVStages * kKvBytes + kSmemExchange;
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kSmemTiles + kSmemExchange + 8 * kNumBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmemTiles + kSmemExchange + 8 * kNumBars + 8);
  auto bar = [&](int which) { return bars + 8u * (uint32_t)which; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x;
  const int kvh = h / (nq / nkv);

  // Which sequence and which 256 rows of it this block owns.  Blocks start in the order of their index,
  // heads fastest: the last rows of every head first (later rows of a prompt see more keys and take
  // longer), the first rows of every head last, so that the short blocks fill the gaps the long ones leave.
  int tile = (int)(gridDim.y - 1 - blockIdx.y), seq = -1, q0 = 0, rows = 0;
  for (int s = 0; s < n_seqs; ++s) {
    const int begin = seq_starts[s], len = seq_starts[s + 1] - begin;
    const int n_tiles = (len + kRowsPerBlock - 1) / kRowsPerBlock;
    if (tile < n_tiles) { seq = s; q0 = begin + tile * kRowsPerBlock; rows = min(kRowsPerBlock, len - tile * kRowsPerBlock); break; }
    tile -= n_tiles;
  }
  if (seq < 0) return;  // the grid was sized with an upper bound
  if (*reinterpret_cast<volatile int*>(status) != 0) return;  // an earlier block gave up: do not pile on
  const int* bt = block_tables + (size_t)seq * max_pages;

  if (tid == 0) {
    for (int s = 0; s < kKStages; ++s) { mbar_init(bar(kBarKFull + s), 1); mbar_init(bar(kBarKEmpty + s), 1); }
    for (int s = 0; s < kVStages; ++s) { mbar_init(bar(kBarVFull + s), 1); mbar_init(bar(kBarVEmpty + s), 1); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(kBarSFull + t), 1);
      mbar_init(bar(kBarPFull + t), kGroupThreads / 32);   // one arrival per warp of the group
      mbar_init(bar(kBarPvDone + t), 1);
    }
    *s_abort = 0;
    mbar_init_fence();
  }
  if (warp == kIssueWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  chain_wait();     // q, positions and this step's keys and values are written by the kernels before this one

  const int pos0 = positions[q0];                       // position of the block's first row
  const int last_key = pos0 + rows - 1;                 // the last key any row of the block sees
  const int rows_t[2] = {min(rows, BM), max(rows - BM, 0)};
  // key tiles each query tile walks: up to the tile that holds its last row's own key
  const int n_t[2] = {(pos0 + rows_t[0] - 1) / BN + 1, rows_t[1] > 0 ? last_key / BN + 1 : 0};
  const int n_kv = max(n_t[0], n_t[1]);
  // The last key tile holds `valid_last` keys; the second product stops at the 16 keys that hold the last one.
  const int valid_last = last_key - (n_kv - 1) * BN + 1;
  const int ksteps_last = (valid_last + 15) >> 4;
  // This block's range of key tiles [j0, j1) (all of them without splits), and where each query tile stops in it.
  const int per_split = (n_kv + key_splits - 1) / key_splits;
  const int j0 = (int)blockIdx.z * per_split, j1 = min(n_kv, j0 + per_split);
  const int n_end[2] = {min(n_t[0], j1), min(n_t[1], j1)};

  if (warp < kSoftmaxWarps) {
    // Q tiles: each softmax thread copies its share (a warp covers whole 128-byte rows); rows past the
    // portion's end are zeros.
    const int lc = tid & 7, lr = tid >> 3;              // 64 rows per pass of the 512 threads
#pragma unroll
    for (int i = 0; i < kRowsPerBlock / 64; ++i) {
      const int r = lr + 64 * i;
      const bool valid = r < rows;
      const __nv_bfloat16* src = q + (size_t)(q0 + (valid ? r : 0)) * q_row_stride + (size_t)h * HD + lc * 8;
      cp_async16(sQ + (r >> 7) * kQBytes + swz(r & (BM - 1), lc), src, valid);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_proxy();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  int copies_k = 0, copies_v = 0;       // key and value tiles the copy warp has asked for

  if (warp == kCopyWarp) {
    // ---- the copy warp: lane i brings page i of a tile; up to four K tiles and four V tiles are in flight ----
    const int pages_per_tile = BN / page_size;
    const uint32_t page_bytes = (uint32_t)page_size * 128u;
    bool ok = true;
    auto wait = [&](int which, uint32_t parity) {      // the first lane polls, the others sleep in the vote
      bool mine = true;
      if (lane == 0) mine = mbar_wait_or_abort(bar(which), parity, s_abort);
      return __all_sync(0xffffffffu, mine) != 0;
    };
    // The page a lane brings is read from the block table one tile ahead, so that the latency of that
    // load is not in the way of the copies.
    auto page_of = [&](int j) {
      const int first_key = j * BN + lane * page_size;
      return (j < n_kv && lane < pages_per_tile && first_key <= last_key) ? bt[first_key / page_size] : -1;
    };
    auto bring = [&](int j, int page, const CUtensorMap* map, uint32_t dst, uint32_t full) {
      const int n_pages = min(pages_per_tile, (last_key - j * BN) / page_size + 1);
      if (lane == 0) mbar_expect(full, (uint32_t)n_pages * page_bytes);
      __syncwarp();
      if (page >= 0) tma_load_rows(dst + (uint32_t)lane * page_bytes, map, (page * nkv + kvh) * page_size, full);
    };
    int page_next = page_of(j0);
    for (int j = j0; j < j1 && ok; ++j) {
      const int jj = j - j0;                            // stages and barrier phases count from the block's first tile
      const int ks = jj & (kKStages - 1), vs = jj & (kVStages - 1);
      const int page = page_next;
      page_next = page_of(j + 1);
      if (jj >= kKStages) ok = wait(kBarKEmpty + ks, ((jj / kKStages) - 1) & 1);
      if (!ok) break;
      bring(j, page, &map_k, sK + ks * kKvBytes, bar(kBarKFull + ks));
      copies_k = jj + 1;
      if (jj >= kVStages) ok = wait(kBarVEmpty + vs, ((jj / kVStages) - 1) & 1);
      if (!ok) break;
      bring(j, page, &map_v, sV + vs * kKvBytes, bar(kBarVFull + vs));
      copies_v = jj + 1;
    }
  } else if (warp == kIssueWarp) {
    // ---- one thread issues the products (a lone thread runs an instruction every few clocks: its code is kept short) ----
    if (lane == 0 && j0 < j1) {
      const uint64_t dq[2] = {make_desc(sQ), make_desc(sQ + kQBytes)};
      const uint64_t dk0 = make_desc(sK), dv0 = make_desc(sV);
      const uint32_t d_s[2] = {tmem + kColS, tmem + kColS + BN}, d_o[2] = {tmem + kColO, tmem + kColO + HD},
                     a_p[2] = {tmem + kColP, tmem + kColP + BN / 2};
      bool ok = true;
      auto issue_s = [&](int t, int j) {                // S_t(j) = Q_t K(j)^T
        const uint64_t dk = dk0 + (uint64_t)(((j - j0) & (kKStages - 1)) * (kKvBytes >> 4));
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) mma_bf16(d_s[t], dq[t] + 2 * k, dk + 2 * k, kIdescS, k > 0);
        mma_commit(bar(kBarSFull + t));
      };
      auto issue_pv = [&](int t, int j) {               // O_t += P_t(j) V(j): 16 keys per step, 8 columns of P, 2048 bytes of V
        const uint64_t dv = dv0 + (uint64_t)(((j - j0) & (kVStages - 1)) * (kKvBytes >> 4));
        if (j < n_kv - 1) {
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            mma_bf16_a_tmem(d_o[t], a_p[t] + k * 8, dv + (uint64_t)(k * (2048 >> 4)), kIdescO, (j > j0 || k > 0) ? 1u : 0u);
        } else {
          for (int k = 0; k < ksteps_last; ++k)
            mma_bf16_a_tmem(d_o[t], a_p[t] + k * 8, dv + (uint64_t)(k * (2048 >> 4)), kIdescO, (j > j0 || k > 0) ? 1u : 0u);
        }
        mma_commit(bar(kBarPvDone + t));
      };
      ok = mbar_wait_or_abort(bar(kBarKFull + 0), 0, s_abort);
      if (ok) {
        if (j0 < n_end[0]) issue_s(0, j0);
        if (j0 < n_end[1]) issue_s(1, j0);
        mma_commit(bar(kBarKEmpty + 0));
      }
      for (int j = j0; j < j1 && ok; ++j) {
        const int jj = j - j0;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= n_end[t]) continue;
          ok = mbar_wait_or_abort(bar(kBarPFull + t), jj & 1, s_abort);   // P_t(j) is written and S_t(j) has been read
          if (!ok) break;
          fence_after_sync();
          if (j + 1 < n_end[t]) {
            const bool first_user = (t == 0) || (j + 1 >= n_end[0]);
            const bool last_user = (t == 1) || (j + 1 >= n_end[1]);
            if (first_user) ok = mbar_wait_or_abort(bar(kBarKFull + ((jj + 1) & (kKStages - 1))), ((jj + 1) / kKStages) & 1, s_abort);
            if (!ok) break;
            issue_s(t, j + 1);
            if (last_user) mma_commit(bar(kBarKEmpty + ((jj + 1) & (kKStages - 1))));
          }
          const bool first_user = (t == 0) || (j >= n_end[0]);
          const bool last_user = (t == 1) || (j >= n_end[1]);
          if (first_user) {
            ok = mbar_wait_or_abort(bar(kBarVFull + (jj & (kVStages - 1))), (jj / kVStages) & 1, s_abort);
            if (!ok) break;
            if (j == n_kv - 1) {
              // Rows behind the last key may hold anything (unwritten slots of the page, an earlier tile):
              // their P is zero, but 0 * NaN would spoil the product, so they are made zero.
              uint8_t* v_tile = smem + (sV - base) + (jj & (kVStages - 1)) * kKvBytes;
              for (int idx = 0; idx < (ksteps_last * 16 - valid_last) * 8; ++idx)
                *reinterpret_cast<uint4*>(v_tile + swz(valid_last + (idx >> 3), idx & 7)) = make_uint4(0, 0, 0, 0);
              fence_async_proxy();
            }
          }
          issue_pv(t, j);
          if (last_user) mma_commit(bar(kBarVEmpty + (jj & (kVStages - 1))));
        }
      }
    }
  } else {
    // ---- the softmax groups: two threads per query row, each with 64 of a tile's 128 keys ----
    // group t: warps 8 t .. 8 t + 7; warp w of the group reaches the TMEM lanes of rows 32 (w & 3) .. + 31
    // and takes the keys 64 (w >> 2) .. + 63 of every tile
    const int t = warp >> 3, quarter = warp & 3, half = (warp >> 2) & 1;
    const int row = quarter * 32 + lane;
    const int my_pos = pos0 + t * BM + row;
    const uint32_t t_lane = tmem + ((uint32_t)(quarter * 32) << 16);      // this warp's 32 lanes of TMEM
    const uint32_t t_s = t_lane + kColS + t * BN + half * 64, t_o = t_lane + kColO + t * HD + half * 32;
    const uint32_t t_p = t_lane + kColP + t * (BN / 2) + half * 32;
    const int pair_barrier = 1 + t * 4 + quarter;                         // the two warps that share these rows
    float* mine = exchange + (t * BM + row) * 2 + half;
    const float* partners = exchange + (t * BM + row) * 2 + (half ^ 1);
    bool ok = true;
    auto wait = [&](int which, uint32_t parity) {
      if (ok) ok = mbar_wait_or_abort(bar(which), parity, s_abort);
      ok = __all_sync(0xffffffffu, ok) != 0;             // the same answer for every lane: TMEM loads are collective
    };
    float m_ref = -INFINITY, l_run = 0.f;                // l_run: this thread's half of the row's sum
    for (int j = j0; j < n_end[t]; ++j) {
      wait(kBarSFull + t, (j - j0) & 1);
      if (!ok) break;
      fence_after_sync();
      const int key0 = j * BN + half * 64;
      const bool diagonal = j * BN + BN - 1 > pos0 + t * BM;             // some row of the tile has masked keys here
      // The exponentials are taken against the reference maximum of the tiles before, without looking
      // for this tile's maximum first: P is a floating-point number, so a reference that is too low by
      // many powers of two costs no precision.  Only when a row's sum shows that the reference is far
      // too low (or on the first tile, which has none) is the maximum searched, the reference moved,
      // O and the running sum rescaled, and the tile's P computed again.
      float l_tile = 0.f;
      uint32_t packed[32];
      bool search = j == j0;
      for (;;) {
        if (search) {
          float m_half = -INFINITY;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            float s[32];
            tmem_ld32(t_s + 32 * c, s);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) m_half = fmaxf(m_half, (diagonal && key0 + 32 * c + i > my_pos) ? -INFINITY : s[i]);
          }
          *mine = m_half;
          named_barrier(pair_barrier, 64);
          // (scale > 0: the maximum of the scaled scores.  A range of keys may begin with a tile of which a row
          // sees nothing: its reference then stays at a finite floor, so that exp2(-inf - reference) is 0, not NaN.)
          const float m_tile = fmaxf(fmaxf(m_half, *partners) * scale_log2, -1e30f);
          float alpha = 1.f;
          if (m_tile > m_ref) {
            alpha = fast_exp2(m_ref - m_tile);                          // 0 on the first tile
            m_ref = m_tile;
          }
          l_run *= alpha;
          if (j > j0) {
            // O is rescaled in TMEM: P V of tile j-1 must have landed first
            wait(kBarPvDone + t, (j - 1 - j0) & 1);
            if (!ok) break;
            fence_after_sync();
            float acc[32];
            tmem_ld32(t_o, acc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] *= alpha;
            tmem_st32(t_o, acc);
          }
        }
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        // 16 keys at a time; the scores of the next 16 are on their way from TMEM while these are
        // exponentiated.  P is collected in registers and stored once at the end, so that the wait for the
        // second product of the tile before (whose P these stores overwrite) comes as late as possible.
        float s[2][16];
        tmem_ld16(t_s, s[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld16(t_s + 16 * (c + 1), s[(c + 1) & 1]);
          float* sc = s[c & 1];
          if (diagonal) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (key0 + 16 * c + i > my_pos) sc[i] = -INFINITY;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float p0 = fast_exp2(fmaf(sc[2 * i], scale_log2, -m_ref));
            const float p1 = fast_exp2(fmaf(sc[2 * i + 1], scale_log2, -m_ref));
            l4[i & 3] += p0 + p1;
            __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
            packed[8 * c + i] = *reinterpret_cast<uint32_t*>(&b);
          }
        }
        l_tile = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        // both threads of a row have to agree on the reference: the two warps decide together
        if (search || !named_barrier_any(pair_barrier, 64, !(l_tile < kSumLimit))) break;
        search = true;
      }
      if (!ok) break;
      if (j > j0) {
        // P V of tile j-1 has to be done before its P is overwritten
        wait(kBarPvDone + t, (j - 1 - j0) & 1);
        if (!ok) break;
        fence_after_sync();
      }
      tmem_st32(t_p, reinterpret_cast<const float*>(packed));
      tmem_st_wait();
      l_run += l_tile;
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull + t));
    }
    // where this row's share of a split goes: [token][head][split] records of HD floats, and of (maximum, sum)
    const size_t record = ((size_t)(q0 + t * BM + row) * nq + h) * key_splits + blockIdx.z;
    if (n_end[t] <= j0) {
      // nothing of this range is visible to this query tile: an empty record for the merge
      if (key_splits > 1 && half == 0 && row < rows_t[t]) { part_ml[record * 2] = -INFINITY; part_ml[record * 2 + 1] = 0.f; }
    } else {
      wait(kBarPvDone + t, (n_end[t] - 1 - j0) & 1);
      fence_after_sync();
      mine[2 * 2 * BM] = l_run;                          // (a slot of its own: the partner may still be reading a maximum)
      named_barrier(pair_barrier, 64);
      if (ok && key_splits > 1) {
        float acc[32];
        tmem_ld32(t_o, acc);
        tmem_ld_wait();
        if (row < rows_t[t]) {
          float4* dst = reinterpret_cast<float4*>(part_o + record * HD + half * 32);
#pragma unroll
          for (int d = 0; d < 8; ++d) dst[d] = make_float4(acc[4 * d], acc[4 * d + 1], acc[4 * d + 2], acc[4 * d + 3]);
          if (half == 0) { part_ml[record * 2] = m_ref; part_ml[record * 2 + 1] = l_run + partners[2 * 2 * BM]; }
        }
      } else if (ok) {
        const float inv = 1.f / (l_run + partners[2 * 2 * BM]);
        __nv_bfloat16* dst = out + (size_t)(q0 + t * BM + row) * out_row_stride + (size_t)h * HD + half * 32;
        float acc[32];
        tmem_ld32(t_o, acc);
        tmem_ld_wait();
        if (row < rows_t[t]) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
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
    }
  }

  fence_before_sync();
  __syncthreads();
  if (*s_abort) {
    // Copies that were asked for may still be on their way: let every tile that was requested land
    // before the shared memory is given back (each wait bounded on its own).
    if (warp == kCopyWarp && lane == 0) {
      for (int i = max(0, copies_k - kKStages); i < copies_k; ++i) mbar_wait(bar(kBarKFull + (i & (kKStages - 1))), (i / kKStages) & 1);
      for (int i = max(0, copies_v - kVStages); i < copies_v; ++i) mbar_wait(bar(kBarVFull + (i & (kVStages - 1))), (i / kVStages) & 1);
    }
    if (tid == 0) atomicCAS(status, 0, 1000000 + (int)(blockIdx.y * gridDim.x + blockIdx.x));
    __syncthreads();
  }
  if (warp == kIssueWarp) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Merges the key ranges of each (token, head): the ranges' reference maxima are in the log2 domain; a
// range that saw no key has sum 0.  One warp per (token, head), a lane for two neighbouring elements.
__global__ void __launch_bounds__(128)
attention_prefill_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                               int out_row_stride, int first_row, int n_rows, int nq, int key_splits) {
  chain_wait();
  const int pair = (int)(blockIdx.x * 4 + (threadIdx.x >> 5)), lane = threadIdx.x & 31;
  if (pair >= n_rows * nq) return;
  const int row = first_row + pair / nq, h = pair % nq;
  const size_t record = ((size_t)row * nq + h) * key_splits;
  float m = -INFINITY;
  for (int s = 0; s < key_splits; ++s) m = fmaxf(m, part_ml[(record + s) * 2]);
  float l = 0.f, o0 = 0.f, o1 = 0.f;
  for (int s = 0; s < key_splits; ++s) {
    const float ls = part_ml[(record + s) * 2 + 1];
    if (ls == 0.f) continue;                              // (its O was never written)
    const float w = exp2f(part_ml[(record + s) * 2] - m);
    const float2 o = *reinterpret_cast<const float2*>(part_o + (record + s) * HD + 2 * lane);
    l += ls * w;
    o0 += o.x * w;
    o1 += o.y * w;
  }
  const float inv = 1.f / l;
  *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row * out_row_stride + (size_t)h * HD + 2 * lane) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
}

}  // namespace

// Rows of one (sequence, head) that a block takes: the caller sizes the grid with it.
ERB_EXPORT int erb_attention_prefill_rows_per_block() { return kRowsPerBlock; }

// Whether erb_attention_prefill_tc takes these sizes (bfloat16 is implied).
ERB_EXPORT int erb_attention_prefill_tc_supported(int head_dim, int page_size) {
  return head_dim == HD && page_size >= 8 && page_size <= BN && (page_size & (page_size - 1)) == 0;
}

// Portions of prompts only (bfloat16, head_dim 64, no window, pages of 8 to 128 tokens, a power of
// two).  q / out: row t is token t of the batch; seq_starts: int32 [n_seqs + 1] token offsets of the
// sequences to process (consecutive rows of block_tables); n_blocks: sum over them of
// ceil(length / 256) (an upper bound is fine); n_pool_pages: pages of k_pages / v_pages (the tensor
// maps cover the whole pool).  status: device int, set non-zero if a block gave up waiting.
// key_splits > 1: every block's key tiles are cut into that many ranges (for portions that are short
// against their past); first_row and n_rows name the rows of q / out that the sequences cover (they
// are consecutive), part_o has room for (first_row + n_rows) * nq * key_splits * 64 floats and part_ml
// for (first_row + n_rows) * nq * key_splits * 2.
ERB_EXPORT int erb_attention_prefill_tc(const void* q, int q_row_stride, const void* k_pages, const void* v_pages,
                                        int n_pool_pages, const int* block_tables, int max_pages,
                                        const int* seq_starts, const int* positions, void* out, int out_row_stride,
                                        int n_seqs, int n_blocks, int nq, int nkv, int head_dim, int page_size,
                                        float scale, int* status, int key_splits, int first_row, int n_rows,
                                        float* part_o, float* part_ml, void* stream) {
  if (n_seqs <= 0 || n_blocks <= 0) return ERB_OK;
  if (key_splits < 1 || key_splits > 64 || (key_splits > 1 && (!part_o || !part_ml || first_row < 0 || n_rows <= 0 || ((uintptr_t)part_o & 15))))
    return fail(ERB_ERR_ARG, "attention_prefill_tc: bad split arguments");
  if (!erb_attention_prefill_tc_supported(head_dim, page_size))
    return fail(ERB_ERR_UNSUPPORTED, "attention_prefill_tc: head_dim %d with pages of %d (takes 64 with 8, 16, 32, 64 or 128)",
                head_dim, page_size);
  if (nq <= 0 || nkv <= 0 || nq % nkv || n_blocks > 65535) return fail(ERB_ERR_ARG, "attention_prefill_tc: bad head counts or too many blocks");
  if (max_pages <= 0 || !status || n_pool_pages <= 0) return fail(ERB_ERR_ARG, "attention_prefill_tc: bad cache arguments");
  if (q_row_stride % 8 || out_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127))
    return fail(ERB_ERR_UNSUPPORTED, "attention_prefill_tc: rows must be 16-byte aligned, pools 128-byte aligned");
  if ((unsigned long long)n_pool_pages * nkv * page_size > 0x7fffffffull)
    return fail(ERB_ERR_UNSUPPORTED, "attention_prefill_tc: pool too large for 32-bit row coordinates");
  const unsigned long long pool_rows = (unsigned long long)n_pool_pages * nkv * page_size;
  CUtensorMap mk, mv;
  int rc;
  if ((rc = pool_map(&mk, k_pages, pool_rows, (unsigned)page_size, "attention_prefill_tc")) ||
      (rc = pool_map(&mv, v_pages, pool_rows, (unsigned)page_size, "attention_prefill_tc")))
    return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);
    if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "attention_prefill_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  launch_chained(attention_prefill_kernel, dim3(nq, n_blocks, key_splits), dim3(kThreads), kSmemBytes, (cudaStream_t)stream, mk, mv,
                 (const __nv_bfloat16*)q, q_row_stride, block_tables, max_pages, seq_starts, positions,
                 (__nv_bfloat16*)out, out_row_stride, n_seqs, nq, nkv, page_size, scale_log2, status, key_splits, part_o, part_ml);
  if ((rc = check_launch("attention_prefill_tc")) || key_splits == 1) return rc;
  launch_chained(attention_prefill_merge_kernel, dim3((n_rows * nq + 3) / 4), dim3(128), 0, (cudaStream_t)stream, part_o, part_ml,
                 (__nv_bfloat16*)out, out_row_stride, first_row, n_rows, nq, key_splits);
  return check_launch("attention_prefill_merge");
}
