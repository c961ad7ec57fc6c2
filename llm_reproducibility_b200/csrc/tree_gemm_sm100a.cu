// Tree-ordered row-split GEMM for sm_100a (B200):  C[M,N] = A[M,K] * W[N,K]^T.
//
// K is cut into leaves of `leaf` elements.  Each leaf is a run of tcgen05.mma (K=16 per
// instruction) into a fresh fp32 TMEM accumulator; the finished leaf is rounded ONCE to the
// input type (bf16 / fp16) and then combined with the other leaves in a fixed tree:
// level 0 sums F consecutive leaves left to right, the levels above are a perfect binary
// tree, every node rounded to the input type.  The order of operations for one output
// element depends only on (K, leaf) -- never on M, on the tile grid or on how many CTAs run --
// so results are bitwise identical across batch sizes, and a K-shard that starts on a subtree
// boundary yields exactly the subtree's root.  This is the reduction the reference's Triton
// kernel performs (src/tbik/tree_based_matmul.py:121-174); here it is laid out for Blackwell:
//
//   warp 0      TMA producer: 128x64 A box + W box per stage, 128-byte swizzle
//   warp 1      UMMA issuer : tcgen05.mma, two accumulators in TMEM (leaf i+1 runs while leaf i drains)
//   warp 2      TMEM allocator (all 512 columns)
//   warps 4-11  epilogue: tcgen05.ld the leaf in 32-column chunks, round, carry-chain combine, store
//
// The tree stack holds one partial tile per level.  Level 0 stays in registers.  The levels above
// go, in this order, to spare TMEM columns (packed 2 x 16 bit per column), to shared memory and --
// only for levels that are touched once every >= 4 leaves -- to a per-CTA slice of a global
// scratch buffer that stays in L2.  Each epilogue thread only ever touches its own stack words.
//
// Tilings (template parameters BN, PAIR); all give identical bits, asserted by the tests:
//   BN=128 single   128x128 tile, UMMA 128x128x16; 256 TMEM columns left for 4 stack levels; no scratch.
//                   Used when there are too few rows for 128x256 tiles to occupy the SMs, or no scratch.
//   BN=64 / BN=32   128x64 and 128x32 tiles for small M (decode): the GEMM then streams W from HBM and
//                   needs every SM pulling; the whole stack fits TMEM.
//   BN=256 single   128x256 tile, UMMA 128x256x16: the instruction shape that runs the tensor core at
//                   full rate and needs 25% less shared-memory traffic per FLOP; the accumulators
//                   fill TMEM, so the stack above level 0 lives in shared memory and scratch.
//   PAIR            a cluster of two CTAs per tile of 256 rows (cta_group::2): each CTA loads its own
//                   128 rows of A and half of the W tile and drains its own half of the accumulator;
//                   the partner CTA tells the leader's UMMA issuer when its half of a stage landed.
#include <cuda.h>
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "ar_common.cuh"
#include "ptx_sm100a.cuh"
#include "tbik_internal.h"

namespace tbik {

// Development aid, off in the shipped library.  Built with -DTBIK_WAIT_PROFILE=1 block 0's UMMA issuer counts the SM
// cycles it waits for a drained accumulator and for a landed pipeline stage; with =2 its first epilogue warp counts
// the cycles it waits for a finished leaf and the cycles from there to releasing the accumulator.  The two counts
// come back as words 1 and 2 of tbik_gemm_status (word 3 is block 0's total, word 0 stays the error code).
#ifndef TBIK_WAIT_PROFILE
#define TBIK_WAIT_PROFILE 0
#endif

constexpr int BM = 128;   // rows of C per CTA
constexpr int BK = 64;    // one 128-byte swizzle row of 16-bit elements
constexpr int UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 384;
constexpr int EPI_WARP0 = 4;
constexpr int NUM_EPI_WARPS = 8;
constexpr int EPI_THREADS = NUM_EPI_WARPS * 32;
constexpr uint32_t TMEM_COLS = 512;
constexpr int CHUNK = 32;  // accumulator columns drained per tcgen05.ld
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
constexpr int kMaxSplits = 16;            // K-slabs per output tile
constexpr size_t kCounterBytes = 16384;   // head of the workspace: one arrival counter per 128-row block of a tile

struct GemmParams {
  void* C;
  int64_t ldc;
  int M, N;
  int kblocks_per_leaf;  // leaf / 64
  int T, F, L;           // leaves per tile, level-0 radix, number of levels
  int tiles_m, tiles_n, group_m;  // tiles_m counts 128-row (single) or 256-row (pair) tiles
  uint32_t* scratch;     // global stack levels: [cta][level][chunk][word][epilogue thread]
  int scratch_levels;    // levels per CTA held in `scratch`
  int tma_store;         // 1: write C with TMA stores staged in the shared-memory stack slot (tmap_c valid)
  int splits;            // K-slabs per output tile (power of two); slab s covers leaves [s*T, (s+1)*T) and writes
  int64_t split_stride;  // its subtree root to C + s * split_stride elements (C = the partial buffer when > 1)
  // K-slabs only: the CTA that stores the last of a tile's `splits` roots adds them and writes the result here
  void* out;
  int64_t ldo;
  int n_out;             // true number of columns (N above is rounded up to 8 for the roots)
  uint32_t* counters;    // arrivals per 128-row block of an output tile; zero before and after every launch
  // Bytes one TMA load of A delivers per stage.  With fewer than 128 rows of A the box covers only 16, 32 or 64
  // rows: the rest of the 128-row shared-memory tile keeps whatever it held, the UMMA multiplies that too, and
  // the rows of C it produces are never stored (a row of C depends on no other row of A).
  uint32_t a_box_bytes;
  // L2 eviction priority of the loads of A and of W (0 normal, 1 evict first, 2 evict last).  Within a group of row
  // tiles every wave of CTAs re-reads the group's rows of A and meets new rows of W; at K = 12288 one wave touches
  // about 79 MB, so under plain LRU a line of A has left L2 by the time the next wave asks for it.
  int hint_a, hint_b;
  uint32_t* status;      // [0] error code, [1] block, [2] role, [3] SM cycles of block 0 (last launch)
};

// Static shape of one kernel variant.
template <int BN, int STAGES, int SLEVELS, bool PAIR>
struct Cfg {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;              // rows of W this CTA loads per stage
  static constexpr uint32_t B_STAGE_BYTES = B_ROWS * BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;              // rows of C per scheduled tile
  static constexpr int EPI_HALVES = BN >= 64 ? 2 : 1;            // warps per TMEM lane quadrant that drain columns
  static constexpr int COLS_PER_WARP = BN / EPI_HALVES;
  static constexpr int NCH = COLS_PER_WARP / CHUNK;              // chunks per thread per leaf
  static constexpr int LEVEL_WORDS = EPI_THREADS * NCH * (CHUNK / 2);  // packed words of one stack level
  static constexpr int TMEM_LEVELS = (static_cast<int>(TMEM_COLS) - 2 * BN) / (BN / 2);
  static constexpr uint32_t TMEM_STACK_COL0 = 2 * BN;
  // shared memory map (offsets from a 1024-byte aligned base)
  static constexpr uint32_t OFF_STACK = STAGES * STAGE_BYTES;
  // Variants without stack levels in shared memory get a buffer of their own for staging the finished tile of C
  // (for the TMA stores) when it fits beside the pipeline; the others stage in the slot of stack level 1.
  static constexpr uint32_t STAGING_BYTES =
      (SLEVELS == 0 && BN >= 128 && STAGES * STAGE_BYTES + BM * BN * 2 + 2048 <= 232448) ? BM * BN * 2 : 0;
  static constexpr uint32_t OFF_FULL = OFF_STACK + (SLEVELS > 0 ? SLEVELS * LEVEL_WORDS * 4 : STAGING_BYTES);
  static constexpr uint32_t OFF_EMPTY = OFF_FULL + 8 * STAGES;
  static constexpr uint32_t OFF_TFULL = OFF_EMPTY + 8 * STAGES;
  static constexpr uint32_t OFF_TEMPTY = OFF_TFULL + 16;
  static constexpr uint32_t OFF_EPI_BAR = OFF_TEMPTY + 16;   // rendezvous of the 8 epilogue warps
  static constexpr uint32_t OFF_TMEM_PTR = OFF_EPI_BAR + 8;
  static constexpr uint32_t OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr uint32_t OFF_ARRIVE = OFF_ABORT + 4;          // K-slabs: this CTA's arrival number at its tile
  static constexpr uint32_t SMEM_BYTES = OFF_ARRIVE + 4 + 1024;  // + slack for the manual alignment
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "BN");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

TBIK_DEVICE void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  const int group_size = p.group_m * p.tiles_n;
  const int group_id = tile / group_size;
  const int first_m = group_id * p.group_m;
  const int gsz = min(p.tiles_m - first_m, p.group_m);
  const int local = tile - group_id * group_size;
  tm = first_m + local % gsz;
  tn = local / gsz;
}

// K-slabs: the upper levels of the tree.  `part` holds S subtree roots of one output element row by row
// ([slab][row][column]); the result is their pairwise sum ((r0+r1)+(r2+r3))+..., every add rounded to the element
// type -- the same nodes one CTA would have formed had it walked the whole of K, and the same arithmetic the
// rank-pair tree all-reduce applies to tensor-parallel shards.  One thread handles `packs` consecutive 16-byte
// packs of one row.  The roots were written by other CTAs of this launch: they are read past L1.
template <typename T, int S>
TBIK_DEVICE void combine_roots(const GemmParams& p, int row, int col0, int packs, bool vec_out) {
  const uint4* part = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.C) + static_cast<int64_t>(row) * p.ldc);
  const int64_t slab_packs = p.split_stride / 8;
  T* orow = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(row) * p.ldo;
  constexpr int G = S < 8 ? S : 8;  // roots loaded at a time: a pairwise tree over 16 is the sum of two trees over 8
  for (int k = 0; k < packs; ++k) {
    const int c = col0 + 8 * k;
    if (c >= p.N) break;  // p.N is a multiple of 8: a pack is inside the roots' row or outside as a whole
    uint4 acc = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int g = 0; g < S / G; ++g) {
      uint4 v[G];
#pragma unroll
      for (int sl = 0; sl < G; ++sl) v[sl] = __ldcg(part + (g * G + sl) * slab_packs + c / 8);
#pragma unroll
      for (int stride = 1; stride < G; stride *= 2) {
#pragma unroll
        for (int i = 0; i + stride < G; i += 2 * stride) v[i] = Elem<T>::add(v[i], v[i + stride]);
      }
      acc = g == 0 ? v[0] : Elem<T>::add(acc, v[0]);
    }
    if (vec_out && c + 8 <= p.n_out) {
      *reinterpret_cast<uint4*>(orow + c) = acc;
    } else {
      const uint32_t w[4] = {acc.x, acc.y, acc.z, acc.w};
      uint16_t* d16 = reinterpret_cast<uint16_t*>(orow + c);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c + j < p.n_out) d16[j] = static_cast<uint16_t>(j & 1 ? w[j >> 1] >> 16 : w[j >> 1] & 0xFFFFu);
    }
  }
}

// SLABS: the instantiation that serves K-slab launches (p.splits > 1); the plain one carries none of that code.
// NODE32: tree nodes stay fp32 (leaves are not rounded, every node is one fp32 add, the stack lives in tensor memory
// as fp32 columns); OUT32: the root is stored as fp32 (a rank's subtree root on its way to the cross-rank levels),
// otherwise it is rounded once to the operand type.
template <typename T, int BN, int STAGES, int SLEVELS, bool PAIR, bool SLABS, bool NODE32 = false, bool OUT32 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tree_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using C_ = Cfg<BN, STAGES, SLEVELS, PAIR>;
  constexpr uint32_t STAGE_BYTES = C_::STAGE_BYTES;
  constexpr int TILE_M = C_::TILE_M;
  constexpr int NCH = C_::NCH;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n * p.splits;  // work items: (output tile, K-slab)
  // scheduling unit: a CTA, or a pair of CTAs (cluster of 2) working on one 256-row tile
  const int gemm_ctas = static_cast<int>(gridDim.x);
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_units = PAIR ? gemm_ctas >> 1 : gemm_ctas;
  const bool leader = cta_rank == 0u;

  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + C_::OFF_ABORT);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + C_::OFF_TMEM_PTR);
  auto full_bar = [&](int s) { return smem_base + C_::OFF_FULL + 8u * s; };
  auto empty_bar = [&](int s) { return smem_base + C_::OFF_EMPTY + 8u * s; };
  auto tfull_bar = [&](int a) { return smem_base + C_::OFF_TFULL + 8u * a; };
  auto tempty_bar = [&](int a) { return smem_base + C_::OFF_TEMPTY + 8u * a; };

  if constexpr (PAIR) cluster_sync_all();  // both CTAs of the pair are resident before TMEM is shared

  if (threadIdx.x == 0) {
    *abort_flag = 0u;
    for (int s = 0; s < STAGES; ++s) {
      // pair, leader: its own producer + the partner's "my half has landed" relay
      mbar_init(full_bar(s), (PAIR && leader) ? 2 : 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), PAIR ? 2 * NUM_EPI_WARPS : NUM_EPI_WARPS);  // pair: both CTAs' warps, on the leader's
    }
    mbar_init(smem_base + C_::OFF_EPI_BAR, NUM_EPI_WARPS);
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_base + C_::OFF_TMEM_PTR, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_base + C_::OFF_TMEM_PTR, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  int role_failed = 0;  // which role observed the abort (for the status word)
  const long long cycles0 = clock64();

  // The 256x256 pair tile with nodes of the operand type: its accumulators fill tensor memory, so the epilogue keeps
  // TWO level-0 groups in registers (stack level 1 never leaves them) and needs more registers than a 384-thread
  // launch hands out evenly: the producer / issuer warpgroup gives up what it does not use.
  constexpr bool TWOGROUP = BN == 256 && PAIR && !SLABS && !NODE32;

  if (warp < EPI_WARP0) {
  if constexpr (TWOGROUP) setmaxnreg_dec<56>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA)
    // elect.sync, not lane == 0: the compiler then knows that one thread runs the branch and feeds the TMA
    // and UMMA instructions from uniform registers directly, instead of looping over the active lanes
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      const int kblocks = p.T * p.kblocks_per_leaf;
      bool ok = true;
      const uint64_t pol_a = l2_policy(p.hint_a), pol_b = l2_policy(p.hint_b);
      for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
        int tm, tn;
        tile_coords(p, tile / p.splits, tm, tn);
        const int kb0 = (tile % p.splits) * kblocks;                                       // first k-block of the slab
        const int row0 = tm * TILE_M + static_cast<int>(cta_rank) * BM;                   // this CTA's rows of A
        const int wrow0 = tn * BN + (PAIR ? static_cast<int>(cta_rank) * C_::B_ROWS : 0);  // its rows of W
        // one 64-wide k-block: wait for a free stage, arm its barrier, two tiled loads
        auto load_kblock = [&](int kb) -> bool {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            role_failed = 1;
            return false;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          // every CTA tracks its own bytes on its own barrier
          mbar_arrive_expect_tx(full_bar(stage), p.a_box_bytes + C_::B_STAGE_BYTES);
          tma_load_2d_hint(sa, &tmap_a, (kb0 + kb) * BK, row0, full_bar(stage), pol_a);
          tma_load_2d_hint(sa + A_STAGE_BYTES, &tmap_b, (kb0 + kb) * BK, wrow0, full_bar(stage), pol_b);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          return true;
        };
        if ((kblocks & 3) == 0) {
          // straight-line code for four k-blocks: a taken branch per k-block costs more than issuing its loads
          for (int kb = 0; ok && kb < kblocks; kb += 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (!load_kblock(kb + u)) break;
            }
          }
        } else {
          for (int kb = 0; kb < kblocks; ++kb) {
            if (!load_kblock(kb)) break;
          }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA retires.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (PAIR && !leader) {
      // ---------------------------------------------------------- partner CTA: relay "stage landed" to the leader
      if (elect_one()) {
        int stage = 0;
        uint32_t phase = 0;
        const int kblocks = p.T * p.kblocks_per_leaf;
        bool ok = true;
        for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
          for (int kb = 0; kb < kblocks; ++kb) {
            if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              ok = false;
              role_failed = 5;
              break;
            }
            mbar_arrive_cluster(map_to_cta(full_bar(stage), 0));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    } else if (elect_one()) {
      // ---------------------------------------------------------- UMMA issuer (pair: leader CTA only)
      constexpr uint32_t IDESC = umma_idesc_f16(Pack16<T>::kUmmaFmt, TILE_M, BN);
      const uint64_t desc_a0 = umma_desc_sw128_kmajor(smem_base);
      const uint64_t desc_b0 = umma_desc_sw128_kmajor(smem_base + A_STAGE_BYTES);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t leaf_ctr = 0;
      bool ok = true;
#if TBIK_WAIT_PROFILE == 1
      long long w_acc = 0, w_stage = 0;  // cycles block 0's issuer waited for a drained accumulator / a landed stage
#endif
      // completion signal to this CTA's barrier and, for a pair, to the partner's twin barrier
      auto commit = [&](uint32_t bar) {
        if constexpr (PAIR) {
          umma_commit_pair(bar);
          umma_commit_pair(map_to_cta(bar, 1));
        } else {
          umma_commit(bar);
        }
      };
      for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
        for (int leaf = 0; ok && leaf < p.T; ++leaf, ++leaf_ctr) {
          const uint32_t a = leaf_ctr & 1u;
          const uint32_t aphase = (leaf_ctr >> 1) & 1u;
#if TBIK_WAIT_PROFILE == 1
          const long long t_acc = clock64();
#endif
          if (!mbar_wait_bounded(tempty_bar(a), aphase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            role_failed = 2;
            break;
          }
#if TBIK_WAIT_PROFILE == 1
          w_acc += clock64() - t_acc;
#endif
          tc_fence_after_sync();
          const uint32_t tmem_d = tmem_base + a * BN;
          // one 64-wide k-block: wait for its stage, four UMMAs, release the stage
          auto kblock = [&](int kb) -> bool {
#if TBIK_WAIT_PROFILE == 1
            const long long t_stage = clock64();
#endif
            if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              ok = false;
              role_failed = 3;
              return false;
            }
#if TBIK_WAIT_PROFILE == 1
            w_stage += clock64() - t_stage;
#endif
            tc_fence_after_sync();
            const uint64_t sd = static_cast<uint64_t>(stage) * (STAGE_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t koff = static_cast<uint64_t>(k) * ((UMMA_K * 2) >> 4);
              if constexpr (PAIR)
                umma_f16_ss_pair(tmem_d, desc_a0 + sd + koff, desc_b0 + sd + koff, IDESC, (kb | k) != 0 ? 1u : 0u);
              else
                umma_f16_ss(tmem_d, desc_a0 + sd + koff, desc_b0 + sd + koff, IDESC, (kb | k) != 0 ? 1u : 0u);
            }
            commit(empty_bar(stage));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            return true;
          };
          if (p.kblocks_per_leaf == 4) {
            // the usual leaf of 256: straight-line code, a taken branch per k-block costs more than its UMMAs
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              if (!kblock(kb)) break;
            }
          } else if ((p.kblocks_per_leaf & 3) == 0) {
            // long leaves (fp32 nodes): four k-blocks of straight-line code per trip
            for (int kb4 = 0; ok && kb4 < p.kblocks_per_leaf; kb4 += 4) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (!kblock(kb4 + u)) break;
              }
            }
          } else {
            for (int kb = 0; kb < p.kblocks_per_leaf; ++kb) {
              if (!kblock(kb)) break;
            }
          }
          if (ok) commit(tfull_bar(a));
        }
      }
#if TBIK_WAIT_PROFILE == 1
      if (blockIdx.x == 0 && p.status != nullptr) {
        p.status[1] = static_cast<uint32_t>(w_acc);
        p.status[2] = static_cast<uint32_t>(w_stage);
      }
#endif
    }
  }
  } else {
    // ------------------------------------------------------------ epilogue: drain + tree combine
    if constexpr (TWOGROUP) setmaxnreg_inc<224>();
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    const int h = (warp - EPI_WARP0) >> 2;  // which half of the accumulator's columns
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const int epi_tid = (warp - EPI_WARP0) * 32 + lane;
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
    uint32_t* smem_stack = reinterpret_cast<uint32_t*>(smem_gen + C_::OFF_STACK);
    uint32_t* gl_stack = p.scratch + static_cast<size_t>(blockIdx.x) * p.scratch_levels * C_::LEVEL_WORDS;
    // "accumulator drained" goes to the UMMA issuer, which lives in the leader CTA
    const uint32_t tempty0 = PAIR ? map_to_cta(tempty_bar(0), 0) : tempty_bar(0);

    constexpr int NW = NCH * (CHUNK / 2);  // packed words of one stack level held by one thread
    // Stack level `lvl` (>= 1) of this thread: all NW words at once, so that one memory latency
    // is paid per level, not per chunk.
    auto stack_load = [&](int lvl, uint32_t (&t)[NW]) {
      const int idx = lvl - 1;
      if (idx < C_::TMEM_LEVELS) {
        const uint32_t col = tmem_base + lane_off + C_::TMEM_STACK_COL0 + idx * (BN / 2) + h * (C_::COLS_PER_WARP / 2);
        if constexpr (NW == 16) {
          tmem_ld16(col, *reinterpret_cast<uint32_t(*)[16]>(&t[0]));
        } else {
#pragma unroll
          for (int w = 0; w < NW / 32; ++w) tmem_ld32(col + w * 32, *reinterpret_cast<uint32_t(*)[32]>(&t[w * 32]));
        }
        tmem_wait_ld();
      } else {
        // shared memory or scratch: 16 bytes per thread per access, a warp touches 512 contiguous bytes
        const uint4* src = idx < C_::TMEM_LEVELS + SLEVELS
            ? reinterpret_cast<const uint4*>(smem_stack + (idx - C_::TMEM_LEVELS) * C_::LEVEL_WORDS)
            : reinterpret_cast<const uint4*>(gl_stack + (idx - C_::TMEM_LEVELS - SLEVELS) * C_::LEVEL_WORDS);
#pragma unroll
        for (int w = 0; w < NW / 4; ++w) {
          const uint4 q4 = src[w * EPI_THREADS + epi_tid];
          t[4 * w] = q4.x;
          t[4 * w + 1] = q4.y;
          t[4 * w + 2] = q4.z;
          t[4 * w + 3] = q4.w;
        }
      }
    };
    // Tensor-memory levels only: ask for level `lvl` without waiting (the caller waits with tmem_wait_ld()).
    auto stack_issue = [&](int lvl, uint32_t (&t)[NW]) {
      const uint32_t col = tmem_base + lane_off + C_::TMEM_STACK_COL0 + (lvl - 1) * (BN / 2) + h * (C_::COLS_PER_WARP / 2);
      if constexpr (NW == 16) {
        tmem_ld16(col, *reinterpret_cast<uint32_t(*)[16]>(&t[0]));
      } else {
#pragma unroll
        for (int w = 0; w < NW / 32; ++w) tmem_ld32(col + w * 32, *reinterpret_cast<uint32_t(*)[32]>(&t[w * 32]));
      }
    };
    auto stack_store = [&](int lvl, const uint32_t (&v)[NW]) {
      const int idx = lvl - 1;
      if (idx < C_::TMEM_LEVELS) {
        const uint32_t col = tmem_base + lane_off + C_::TMEM_STACK_COL0 + idx * (BN / 2) + h * (C_::COLS_PER_WARP / 2);
        if constexpr (NW == 16) {
          tmem_st16(col, *reinterpret_cast<const uint32_t(*)[16]>(&v[0]));
        } else {
#pragma unroll
          for (int w = 0; w < NW / 32; ++w) tmem_st32(col + w * 32, *reinterpret_cast<const uint32_t(*)[32]>(&v[w * 32]));
        }
      } else {
        uint4* dst = idx < C_::TMEM_LEVELS + SLEVELS
            ? reinterpret_cast<uint4*>(smem_stack + (idx - C_::TMEM_LEVELS) * C_::LEVEL_WORDS)
            : reinterpret_cast<uint4*>(gl_stack + (idx - C_::TMEM_LEVELS - SLEVELS) * C_::LEVEL_WORDS);
#pragma unroll
        for (int w = 0; w < NW / 4; ++w)
          dst[w * EPI_THREADS + epi_tid] = make_uint4(v[4 * w], v[4 * w + 1], v[4 * w + 2], v[4 * w + 3]);
      }
    };

    // C leaves through the TMA unit when possible: the finished tile is staged (128-byte swizzle) in shared memory
    // -- in a buffer of its own, or in the slot of stack level 1, which is free once the tree is complete -- and one
    // thread issues one tiled store per 64 columns.  The buffer may only be rewritten after those stores have read
    // it.  (Storing the root from registers instead costs a 256x128 tile about 2200 cycles, a tenth of its time at
    // K = 4096: every store instruction of a warp touches 32 rows of C.)
    const bool tma_c = (SLEVELS > 0 || C_::STAGING_BYTES > 0) && p.tma_store != 0;
    bool staging_busy = false;
    bool ok = true;
    uint32_t epi_phase = 0;
    // Rendezvous of the eight epilogue warps on an mbarrier with a bounded wait (a plain bar.sync would
    // wait forever for a warp that has left after an abort).  Every lane waits on the barrier itself: a
    // variant in which lane 0 polled and handed the outcome to the others with a shuffle left lanes 1..31
    // without an acquire, and in a CTA pair the staged tile was then read or rewritten too early (torn
    // 16-byte words in C at four leaves per tile).
    auto epi_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_base + C_::OFF_EPI_BAR);
      if (!mbar_wait_bounded(smem_base + C_::OFF_EPI_BAR, epi_phase, abort_flag, WAIT_LIMIT_NS)) {
        ok = false;
        role_failed = 6;
      }
      epi_phase ^= 1u;
    };
    auto staging_release = [&]() {
      if (staging_busy) {
        if (epi_tid == 0) bulk_wait_read_all();
        epi_sync();
        staging_busy = false;
      }
    };

    // The finished tile of C (this thread's NW packed words of its row) to shared memory, then out with TMA stores.
    // Every epilogue thread calls it, also those whose row lies beyond M: the stores clip.
    auto stage_root = [&](const uint32_t (&v)[NW], int tm, int tn) {
      staging_release();
      // a stack slot is laid out per thread as a stack level but per row as a staged tile: nobody may
      // write tile rows into it before every warp has popped its own level-1 words
      if constexpr (SLEVELS > 0) epi_sync();
      constexpr int CCH = C_::COLS_PER_WARP / 64;  // 64-column boxes per warp
      const int r = q * 32 + lane;
#pragma unroll
      for (int cc = 0; cc < CCH; ++cc) {
        uint8_t* box = reinterpret_cast<uint8_t*>(smem_stack) + (h * CCH + cc) * (BM * 128) + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(box + ((u ^ (r & 7)) << 4)) =
              make_uint4(v[cc * 32 + 4 * u], v[cc * 32 + 4 * u + 1], v[cc * 32 + 4 * u + 2], v[cc * 32 + 4 * u + 3]);
      }
      fence_proxy_async_smem();
      epi_sync();
      if (ok && epi_tid == 0) {
        const uint32_t sbase = smem_base + C_::OFF_STACK;
        const int row0 = tm * TILE_M + static_cast<int>(cta_rank) * BM;
#pragma unroll
        for (int b = 0; b < BN / 64; ++b) tma_store_2d(&tmap_c, sbase + b * (BM * 128), tn * BN + b * 64, row0);
        bulk_commit_group();
      }
      staging_busy = true;
    };

    if (h >= C_::EPI_HALVES) {
      // narrow tiles: this warp has no columns to drain; it only keeps the accumulator hand-shake going
      uint32_t ctr = 0;
      for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
        for (int leaf = 0; ok && leaf < p.T; ++leaf, ++ctr) {
          const uint32_t a = ctr & 1u;
          if (!mbar_wait_bounded(tfull_bar(a), (ctr >> 1) & 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            role_failed = 4;
            break;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * a);
        }
        if (SLABS && ok && p.splits > 1) {
          // keep step with the two rendezvous of the draining warps' arrival protocol (below)
          epi_sync();
          if (ok) epi_sync();
        }
      }
    } else if constexpr (NODE32) {
      // ---------------------------------------------------------- fp32 nodes: nothing is rounded before the root
      constexpr int CW = C_::COLS_PER_WARP;
      float s0f[CW];  // the open level-0 group / the node that climbs the tree, fp32
      auto stack_col = [&](int lvl, int c) -> uint32_t {
        return tmem_base + lane_off + C_::TMEM_STACK_COL0 + static_cast<uint32_t>(lvl - 1) * BN + h * CW + c * CHUNK;
      };
      uint32_t leaf_ctr = 0;
      for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int row = tm * TILE_M + static_cast<int>(cta_rank) * BM + q * 32 + lane;
        int c0 = 0;
        uint32_t g = 0;
        for (int leaf = 0; ok && leaf < p.T; ++leaf, ++leaf_ctr) {
          const uint32_t a = leaf_ctr & 1u;
          const uint32_t aphase = (leaf_ctr >> 1) & 1u;
          if (!mbar_wait_bounded(tfull_bar(a), aphase, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            role_failed = 4;
            break;
          }
          tc_fence_after_sync();
          tmem_wait_st();  // stack stores of earlier leaves have landed
          const uint32_t tacc = tmem_base + lane_off + a * BN + h * CW;
          const bool add0 = c0 > 0;
          {
            uint32_t raw[2][32];
            tmem_ld32(tacc, raw[0]);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              tmem_wait_ld();
              if (c + 1 < NCH) {
                tmem_ld32(tacc + (c + 1) * CHUNK, raw[(c + 1) & 1]);
              } else {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * a);  // accumulator may be overwritten now
              }
#pragma unroll
              for (int j = 0; j < CHUNK; ++j) {
                const float v = __uint_as_float(raw[c & 1][j]);
                s0f[c * CHUNK + j] = add0 ? __fadd_rn(s0f[c * CHUNK + j], v) : v;  // level 0: radix F, sequential
              }
            }
          }
          if (++c0 < p.F) continue;
          c0 = 0;
          uint32_t gb = g++;
          int lvl = 1;
          while (lvl < p.L && (gb & 1u)) {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              uint32_t t[32];
              tmem_ld32(stack_col(lvl, c), t);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < CHUNK; ++j) s0f[c * CHUNK + j] = __fadd_rn(__uint_as_float(t[j]), s0f[c * CHUNK + j]);
            }
            gb >>= 1;
            ++lvl;
          }
          if (lvl < p.L) {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              uint32_t t[32];
#pragma unroll
              for (int j = 0; j < CHUNK; ++j) t[j] = __float_as_uint(s0f[c * CHUNK + j]);
              tmem_st32(stack_col(lvl, c), t);
            }
          } else if (!OUT32 && tma_c) {
            // the one rounding of this mode, then out through the staging buffer
            uint32_t w[NW];
#pragma unroll
            for (int j = 0; j < NW; ++j) w[j] = Pack16<T>::from_f32(s0f[2 * j], s0f[2 * j + 1]);
            stage_root(w, tm, tn);
          } else if (row < p.M) {
            // root of the tile's tree
            if constexpr (OUT32) {
              float* crow = reinterpret_cast<float*>(p.C) + static_cast<int64_t>(row) * p.ldc;
              const bool vec32 = (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
#pragma unroll
              for (int c = 0; c < NCH; ++c) {
                const int col0 = tn * BN + h * CW + c * CHUNK;
                if (col0 >= p.N) continue;
                if (vec32 && col0 + CHUNK <= p.N) {
                  float4* dst = reinterpret_cast<float4*>(crow + col0);
#pragma unroll
                  for (int j = 0; j < CHUNK / 4; ++j)
                    dst[j] = make_float4(s0f[c * CHUNK + 4 * j], s0f[c * CHUNK + 4 * j + 1], s0f[c * CHUNK + 4 * j + 2],
                                         s0f[c * CHUNK + 4 * j + 3]);
                } else {
#pragma unroll
                  for (int j = 0; j < CHUNK; ++j)
                    if (col0 + j < p.N) crow[col0 + j] = s0f[c * CHUNK + j];
                }
              }
            } else {
              // the one rounding of this mode
              T* crow = reinterpret_cast<T*>(p.C) + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
              for (int c = 0; c < NCH; ++c) {
                const int col0 = tn * BN + h * CW + c * CHUNK;
                if (col0 >= p.N) continue;
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) w[j] = Pack16<T>::from_f32(s0f[c * CHUNK + 2 * j], s0f[c * CHUNK + 2 * j + 1]);
                if (vec_ok && col0 + CHUNK <= p.N) {
                  uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
                  for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                } else {
                  uint16_t* dst = reinterpret_cast<uint16_t*>(crow + col0);
#pragma unroll
                  for (int j = 0; j < 16; ++j) {
                    if (col0 + 2 * j < p.N) dst[2 * j] = static_cast<uint16_t>(w[j] & 0xFFFFu);
                    if (col0 + 2 * j + 1 < p.N) dst[2 * j + 1] = static_cast<uint16_t>(w[j] >> 16);
                  }
                }
              }
            }
          }
        }
      }
    } else if constexpr (TWOGROUP) {
      // ---------------------------------------------------------- two level-0 groups per trip, level 1 in registers
      // Stack level lvl >= 2 lives in slot lvl - 2: the shared-memory slot first, the scratch after it.
      uint32_t sA[NW], s0[NW];
      uint32_t leaf_ctr = 0;
      // wait for the next leaf and drain it into dst (add0: onto what dst holds -- level 0, radix F, left to right)
      auto drain_leaf = [&](uint32_t (&dst)[NW], bool add0) -> bool {
        const uint32_t a = leaf_ctr & 1u;
        const uint32_t aphase = (leaf_ctr >> 1) & 1u;
        ++leaf_ctr;
        if (!mbar_wait_bounded(tfull_bar(a), aphase, abort_flag, WAIT_LIMIT_NS)) {
          ok = false;
          role_failed = 4;
          return false;
        }
        tc_fence_after_sync();
        const uint32_t tacc = tmem_base + lane_off + a * BN + h * C_::COLS_PER_WARP;
        uint32_t raw[2][32];
        tmem_ld32(tacc, raw[0]);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tmem_wait_ld();
          if (c + 1 < NCH) {
            tmem_ld32(tacc + (c + 1) * CHUNK, raw[(c + 1) & 1]);
          } else {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * a);  // accumulator may be overwritten now
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t v = Pack16<T>::from_f32(__uint_as_float(raw[c & 1][2 * j]), __uint_as_float(raw[c & 1][2 * j + 1]));
            dst[c * 16 + j] = add0 ? Pack16<T>::add(dst[c * 16 + j], v) : v;
          }
        }
        return true;
      };
      for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int row = tm * TILE_M + static_cast<int>(cta_rank) * BM + q * 32 + lane;
        T* crow = reinterpret_cast<T*>(p.C) + static_cast<int64_t>(row) * p.ldc;
        const int supers = p.L >= 2 ? (p.T / p.F) >> 1 : 1;  // a tree of one group has nothing above level 0
        for (int sg = 0; ok && sg < supers; ++sg) {
          if (p.L >= 2) {
            for (int i = 0; ok && i < p.F; ++i) drain_leaf(sA, i > 0);
          }
          for (int i = 0; ok && i < p.F; ++i) drain_leaf(s0, i > 0);
          if (!ok) break;
          int lvl = 1;
          if (p.L >= 2) {
#pragma unroll
            for (int w = 0; w < NW; ++w) s0[w] = Pack16<T>::add(sA[w], s0[w]);  // the level-1 node
            uint32_t gb = static_cast<uint32_t>(sg);
            lvl = 2;
            while (lvl < p.L && (gb & 1u)) {
              uint32_t t[NW];
              stack_load(lvl - 1, t);
#pragma unroll
              for (int w = 0; w < NW; ++w) s0[w] = Pack16<T>::add(t[w], s0[w]);
              gb >>= 1;
              ++lvl;
            }
          }
          if (lvl < p.L) {
            if (lvl == 2) staging_release();  // about to overwrite the slot the last tile of C was staged in
            stack_store(lvl - 1, s0);
          } else if (tma_c) {
            stage_root(s0, tm, tn);
          } else if (row < p.M) {
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              const int col0 = tn * BN + h * C_::COLS_PER_WARP + c * CHUNK;
              if (col0 >= p.N) continue;
              if (vec_ok && col0 + CHUNK <= p.N) {
                uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  dst[j] = make_uint4(s0[c * 16 + 4 * j], s0[c * 16 + 4 * j + 1], s0[c * 16 + 4 * j + 2], s0[c * 16 + 4 * j + 3]);
              } else {
                uint16_t* dst = reinterpret_cast<uint16_t*>(crow + col0);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (col0 + 2 * j < p.N) dst[2 * j] = static_cast<uint16_t>(s0[c * 16 + j] & 0xFFFFu);
                  if (col0 + 2 * j + 1 < p.N) dst[2 * j + 1] = static_cast<uint16_t>(s0[c * 16 + j] >> 16);
                }
              }
            }
          }
        }
      }
    } else {
    uint32_t s0[NW];  // the open level-0 group; once it closes, the node that climbs the tree
    constexpr bool PREFETCH1 = C_::TMEM_LEVELS >= 1 && NW <= 32;
    uint32_t pre1[PREFETCH1 ? NW : 1];  // stack level 1, requested ahead of the drain
    uint32_t leaf_ctr = 0;
#if TBIK_WAIT_PROFILE >= 2
    long long w_full = 0, w_drain = 0;  // cycles this warp waited for a finished leaf / spent until it released it
    [[maybe_unused]] long long t_rel = 0;
#endif
    for (int tile = unit; ok && tile < num_tiles; tile += num_units) {
      int tm, tn;
      tile_coords(p, tile / p.splits, tm, tn);
      const int row = tm * TILE_M + static_cast<int>(cta_rank) * BM + q * 32 + lane;
      T* crow = reinterpret_cast<T*>(p.C) + (tile % p.splits) * p.split_stride + static_cast<int64_t>(row) * p.ldc;
      int c0 = 0;       // leaves already summed into the open level-0 group
      uint32_t g = 0;   // finished level-0 groups of this tile
      for (int leaf = 0; ok && leaf < p.T; ++leaf, ++leaf_ctr) {
        const uint32_t a = leaf_ctr & 1u;
        const uint32_t aphase = (leaf_ctr >> 1) & 1u;
        // A leaf that closes an odd-numbered group meets stack level 1 right after its drain: ask tensor memory for
        // it now, while the leaf is still being multiplied, so that the climb starts with the operand at hand.
        bool have1 = false;
        if constexpr (PREFETCH1) {
          if (c0 + 1 == p.F && (g & 1u) && p.L > 1) {
            tmem_wait_st();  // the store that filled level 1 has landed
            stack_issue(1, pre1);
            have1 = true;
          }
        }
#if TBIK_WAIT_PROFILE == 2
        const long long t_full = clock64();
#endif
#if TBIK_WAIT_PROFILE == 4
        const long long t_leaf0 = clock64();
#endif
        if (!mbar_wait_bounded(tfull_bar(a), aphase, abort_flag, WAIT_LIMIT_NS)) {
          ok = false;
          role_failed = 4;
          break;
        }
#if TBIK_WAIT_PROFILE == 2
        const long long t_got = clock64();
        w_full += t_got - t_full;
#endif
        tc_fence_after_sync();
        if constexpr (C_::TMEM_LEVELS > 0) tmem_wait_st();  // stack stores of earlier leaves have landed
        const uint32_t tacc = tmem_base + lane_off + a * BN + h * C_::COLS_PER_WARP;
        const bool add0 = c0 > 0;
        {
          // drain the accumulator chunk by chunk; the next chunk flies while this one is rounded and added
          uint32_t raw[2][32];
          tmem_ld32(tacc, raw[0]);
          if constexpr (NCH == 2) tmem_ld32(tacc + CHUNK, raw[1]);  // two chunks: both in flight, one wait, release
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if (NCH != 2 || c == 0) tmem_wait_ld();
            if (NCH != 2 && c + 1 < NCH) {
              tmem_ld32(tacc + (c + 1) * CHUNK, raw[(c + 1) & 1]);
            } else if (NCH == 2 ? c == 0 : true) {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * a);  // accumulator may be overwritten now
#if TBIK_WAIT_PROFILE == 2
              w_drain += clock64() - t_got;
#endif
#if TBIK_WAIT_PROFILE == 3
              t_rel = clock64();
#endif
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t v = Pack16<T>::from_f32(__uint_as_float(raw[c & 1][2 * j]), __uint_as_float(raw[c & 1][2 * j + 1]));
              s0[c * 16 + j] = add0 ? Pack16<T>::add(s0[c * 16 + j], v) : v;  // level 0: radix F, sequential
            }
          }
        }
#if TBIK_WAIT_PROFILE == 3
        const long long t_conv = clock64();
        w_full += t_conv - t_rel;  // converting and adding the last chunk after the release
#endif
        if (++c0 < p.F) continue;
        c0 = 0;
        // levels >= 1: binary counter over finished groups
        uint32_t gb = g++;
        int lvl = 1;
        if constexpr (PREFETCH1) {
          if (have1) {  // arrived with the drain's wait
#pragma unroll
            for (int w = 0; w < NW; ++w) s0[w] = Pack16<T>::add(pre1[w], s0[w]);
            gb >>= 1;
            lvl = 2;
          }
        }
        while (lvl < p.L && (gb & 1u)) {
          uint32_t t[NW];
          stack_load(lvl, t);
#pragma unroll
          for (int w = 0; w < NW; ++w) s0[w] = Pack16<T>::add(t[w], s0[w]);
          gb >>= 1;
          ++lvl;
        }
#if TBIK_WAIT_PROFILE == 3
        w_drain += clock64() - t_conv;  // the loads and adds of the climb
#endif
#if TBIK_WAIT_PROFILE == 4
        const long long t_store0 = clock64();
        w_full += t_store0 - t_leaf0;  // whole leaves that closed a group, up to the store
#endif
        if (lvl < p.L) {
          if (lvl - 1 == C_::TMEM_LEVELS) staging_release();  // about to overwrite the staging slot
          stack_store(lvl, s0);
#if TBIK_WAIT_PROFILE == 4
          w_drain += clock64() - t_store0;  // stack stores
#endif
        } else if (tma_c) {
#if TBIK_WAIT_PROFILE == 5
          const long long t_root0 = clock64();
#endif
          stage_root(s0, tm, tn);
#if TBIK_WAIT_PROFILE == 5
          w_full += clock64() - t_root0;  // staged root store
#endif
        } else {
#if TBIK_WAIT_PROFILE == 5
          const long long t_root0 = clock64();
#endif
          if (row < p.M) {
          // root of the tile's tree: write this thread's BN/2 columns of C
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            const int col0 = tn * BN + h * C_::COLS_PER_WARP + c * CHUNK;
            if (col0 >= p.N) continue;
            if (vec_ok && col0 + CHUNK <= p.N) {
              uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dst[j] = make_uint4(s0[c * 16 + 4 * j], s0[c * 16 + 4 * j + 1], s0[c * 16 + 4 * j + 2], s0[c * 16 + 4 * j + 3]);
            } else {
              uint16_t* dst = reinterpret_cast<uint16_t*>(crow + col0);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (col0 + 2 * j < p.N) dst[2 * j] = static_cast<uint16_t>(s0[c * 16 + j] & 0xFFFFu);
                if (col0 + 2 * j + 1 < p.N) dst[2 * j + 1] = static_cast<uint16_t>(s0[c * 16 + j] >> 16);
              }
            }
          }
          }
#if TBIK_WAIT_PROFILE == 5
          w_drain += clock64() - t_root0;  // direct root store
#endif
          if (SLABS && p.splits > 1) {
            // K-slabs: this was one of the tile's `splits` subtree roots.  Count the arrival; the CTA that brings
            // the last root adds all of them in the fixed pairwise order and writes C.  Which CTA that is depends
            // on timing, the sum does not: it is formed from all the roots, in slab order, by one thread per pack.
            __threadfence();  // this thread's words of the root are visible device-wide before the arrival counts
            epi_sync();
            volatile uint32_t* arrive = reinterpret_cast<volatile uint32_t*>(smem_gen + C_::OFF_ARRIVE);
            const uint32_t cidx = static_cast<uint32_t>(tile / p.splits) * (PAIR ? 2u : 1u) + cta_rank;
            if (ok && epi_tid == 0) *arrive = atomicAdd(&p.counters[cidx], 1u);
            if (ok) epi_sync();
            if (ok && *arrive == static_cast<uint32_t>(p.splits) - 1u) {
              __threadfence();  // the other CTAs' roots, published before their arrivals, are visible now
              if (epi_tid == 0) p.counters[cidx] = 0u;  // nobody else counts on this tile in this launch any more
              if (row < p.M) {
                const bool vec_out = (p.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0);
                const int col0 = tn * BN + h * C_::COLS_PER_WARP;
                constexpr int PACKS = C_::COLS_PER_WARP / 8;
                switch (p.splits) {
                  case 2: combine_roots<T, 2>(p, row, col0, PACKS, vec_out); break;
                  case 4: combine_roots<T, 4>(p, row, col0, PACKS, vec_out); break;
                  case 8: combine_roots<T, 8>(p, row, col0, PACKS, vec_out); break;
                  default: combine_roots<T, 16>(p, row, col0, PACKS, vec_out); break;
                }
              }
            }
          }
        }
      }
    }
#if TBIK_WAIT_PROFILE >= 2
    if (blockIdx.x == 0 && warp == EPI_WARP0 && lane == 0 && p.status != nullptr) {
      p.status[1] = static_cast<uint32_t>(w_full);
      p.status[2] = static_cast<uint32_t>(w_drain);
    }
#endif
    }  // draining warps
  }

  // ---------------------------------------------------------------- tear-down
  if (warp == EPI_WARP0 && lane == 0) bulk_wait_read_all();  // staged C tiles have left shared memory
  tc_fence_before_sync();
  __syncwarp();
  if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
  if (role_failed != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, 0u, 1u) == 0u) {
      p.status[1] = blockIdx.x;
      p.status[2] = static_cast<uint32_t>(role_failed);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.status != nullptr)
    p.status[3] = static_cast<uint32_t>(clock64() - cycles0);  // SM cycles block 0 spent in the main loop
  if (warp == 2) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ==================================================================== host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  // initialised once, by whichever thread comes first (C++11 guarantees the others wait)
  static const EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(ptr);
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// Tensor maps are pure functions of (address, extents, stride, box, type): a layer that is called again with the
// same weight and the same activation buffer (every decode step under a serving engine) finds its maps here
// instead of paying three driver calls per launch.  One small direct-mapped table per host thread.
struct TmapKey {
  const void* base;
  int64_t rows, K, ld;
  int box_rows, dtype, swizzle;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows && dtype == o.dtype &&
           swizzle == o.swizzle;
  }
};
struct TmapSlot {
  TmapKey key{};
  CUtensorMap map{};
  bool valid = false;
};
constexpr int kTmapSlots = 256;

// Row-major [rows, K] 16-bit matrix, row stride `ld` elements, box = 64 (K) x `box_rows` rows.
int make_tmap(CUtensorMap* tm, int dtype, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows,
              bool quiet = false, bool swizzle = true) {
  static thread_local TmapSlot cache[kTmapSlots];
  const TmapKey key{base, rows, K, ld, box_rows, dtype, swizzle ? 1 : 0};
  uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
  h ^= static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(K) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(box_rows);
  h ^= h >> 29;
  TmapSlot& slot = cache[h % kTmapSlots];
  if (slot.valid && slot.key == key) {
    *tm = slot.map;
    return TBIK_OK;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(TBIK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == TBIK_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (quiet) return TBIK_ERR_CUDA;
    char msg[160];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld K=%lld ld=%lld)", (int)r,
             (long long)rows, (long long)K, (long long)ld);
    return set_error(TBIK_ERR_CUDA, msg);
  }
  slot.key = key;
  slot.map = *tm;
  slot.valid = true;
  return TBIK_OK;
}

__device__ uint32_t g_gemm_status[4];

constexpr int kMaxDevices = 64;

// Device address of the status word, looked up once per device.
uint32_t* status_address(int dev) {
  static std::atomic<uint32_t*> addr[kMaxDevices];
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  uint32_t* p = addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_gemm_status) != cudaSuccess) return nullptr;
    p = static_cast<uint32_t*>(q);
    addr[dev].store(p, std::memory_order_release);
  }
  return p;
}

template <typename T, int BN, int STAGES, int SLEVELS, bool PAIR, bool SLABS, bool NODE32 = false, bool OUT32 = false>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
           cudaStream_t stream, int dev) {
  using C_ = Cfg<BN, STAGES, SLEVELS, PAIR>;
  // set twice at worst when two threads race on a device's first launch: the call is idempotent
  static std::atomic<bool> configured[kMaxDevices];
  static_assert(!NODE32 || (SLEVELS == 0 && BN <= 128 && !SLABS), "fp32 nodes: the stack lives in tensor memory only");
  auto kernel = tree_gemm_kernel<T, BN, STAGES, SLEVELS, PAIR, SLABS, NODE32, OUT32>;
  if (dev >= 0 && dev < kMaxDevices && !configured[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(C_::SMEM_BYTES));
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(tree_gemm_kernel)");
    configured[dev].store(true, std::memory_order_release);
  }
  if constexpr (PAIR) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = C_::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, p);
    if (e != cudaSuccess) return set_cuda_error(e, "tree_gemm_kernel launch");
  } else {
    kernel<<<grid, NUM_THREADS, C_::SMEM_BYTES, stream>>>(ta, tb, tc, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_cuda_error(e, "tree_gemm_kernel launch");
  }
  return TBIK_OK;
}

template <typename T, int BN, int STAGES, int SLEVELS, bool PAIR>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
           cudaStream_t stream, int dev) {
  return p.splits > 1 ? launch_one<T, BN, STAGES, SLEVELS, PAIR, true>(ta, tb, tc, p, grid, stream, dev)
                      : launch_one<T, BN, STAGES, SLEVELS, PAIR, false>(ta, tb, tc, p, grid, stream, dev);
}

// The compiled variants.  `levels_on_chip` = stack levels above level 0 that fit TMEM + shared memory.
struct Variant {
  int bn;
  bool pair;
  int levels_on_chip;
  int level_bytes;  // bytes of one stack level of one CTA
};

template <int BN, int STAGES, int SLEVELS, bool PAIR>
constexpr Variant variant_of() {
  using C_ = Cfg<BN, STAGES, SLEVELS, PAIR>;
  return Variant{BN, PAIR, C_::TMEM_LEVELS + SLEVELS, C_::LEVEL_WORDS * 4};
}

// tiling code -> (shallow, deep) variants; the deep one trades pipeline stages for stack levels
constexpr Variant kVariants[6][2] = {
    {variant_of<128, 6, 0, false>(), variant_of<128, 4, 2, false>()},
    {variant_of<128, 8, 0, true>(), variant_of<128, 5, 2, true>()},
    {variant_of<256, 3, 1, false>(), variant_of<256, 3, 1, false>()},
    {variant_of<256, 5, 1, true>(), variant_of<256, 5, 1, true>()},
    {variant_of<64, 8, 0, false>(), variant_of<64, 8, 0, false>()},
    {variant_of<32, 8, 0, false>(), variant_of<32, 8, 0, false>()},
};

template <typename T>
int launch_variant(int tiling, bool deep, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                   const GemmParams& p, int grid, cudaStream_t stream, int dev) {
  switch (tiling) {
    case 1: return deep ? launch<T, 128, 4, 2, false>(ta, tb, tc, p, grid, stream, dev) : launch<T, 128, 6, 0, false>(ta, tb, tc, p, grid, stream, dev);
    case 2: return deep ? launch<T, 128, 5, 2, true>(ta, tb, tc, p, grid, stream, dev) : launch<T, 128, 8, 0, true>(ta, tb, tc, p, grid, stream, dev);
    case 3: return launch<T, 256, 3, 1, false>(ta, tb, tc, p, grid, stream, dev);
    case 4: return launch<T, 256, 5, 1, true>(ta, tb, tc, p, grid, stream, dev);
    case 5: return launch<T, 64, 8, 0, false>(ta, tb, tc, p, grid, stream, dev);
    case 6: return launch<T, 32, 8, 0, false>(ta, tb, tc, p, grid, stream, dev);
    default: return set_error(TBIK_ERR_ARG, "unknown tiling");
  }
}

// fp32-node launches: the shallow variants of the 128-, 64- and 32-column tilings (their stack fits tensor memory)
template <typename T, bool OUT32>
int launch_node32(int tiling, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                  int grid, cudaStream_t stream, int dev) {
  switch (tiling) {
    case 1: return launch_one<T, 128, 6, 0, false, false, true, OUT32>(ta, tb, tc, p, grid, stream, dev);
    case 2: return launch_one<T, 128, 8, 0, true, false, true, OUT32>(ta, tb, tc, p, grid, stream, dev);
    case 5: return launch_one<T, 64, 8, 0, false, false, true, OUT32>(ta, tb, tc, p, grid, stream, dev);
    case 6: return launch_one<T, 32, 8, 0, false, false, true, OUT32>(ta, tb, tc, p, grid, stream, dev);
    default: return set_error(TBIK_ERR_ARG, "fp32 nodes: tiling must be 1, 2, 5 or 6");
  }
}

int sm_count(int dev) {
  static std::atomic<int> cached[kMaxDevices];
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    // without a device (plan queries on a build machine) answer for the GPU this library is written for
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148;
    }
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

}  // namespace

int tree_shape(int64_t K, int leaf, int* T, int* F, int* L) {
  if (leaf <= 0 || K <= 0 || K % leaf != 0) return TBIK_ERR_SHAPE;
  int64_t t = K / leaf;
  int64_t f = t;
  int l = 1;
  while (f > 2 && f % 2 == 0) {
    f /= 2;
    ++l;
  }
  *T = static_cast<int>(t);
  *F = static_cast<int>(f);
  *L = l;
  return TBIK_OK;
}

// Schedule for one call: which variant, how many CTAs, how much scratch.
// Workspace layout: [arrival counters, kCounterBytes, only with K-slabs][global stack levels][slab roots].
struct Plan {
  int tiling;  // 1..6
  bool deep;
  int grid;
  int tiles_m, tiles_n;
  int splits;             // K-slabs per output tile (1 = the whole tree in one CTA)
  int slab_levels;        // tree levels one work item climbs: L - log2(splits)
  int scratch_levels;
  size_t scratch_off;     // offset of the global stack levels in the workspace
  size_t scratch_bytes;   // global stack levels
  size_t partial_off;     // offset of the slab roots in the workspace (0 when splits == 1)
  size_t partial_bytes;   // [splits][M][N rounded up to 8] elements
  bool valid;
  size_t total_bytes() const {
    if (splits > 1) return partial_off + partial_bytes;
    return scratch_bytes > 0 ? scratch_off + scratch_bytes : 0;
  }
};

static int log2_int(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

// `L` is the depth of the whole tree; with `splits` > 1 each work item climbs only the lower L - log2(splits) levels.
static Plan make_plan(int tiling, int M, int N, int L, int max_ctas, int splits = 1) {
  Plan pl{};
  pl.tiling = tiling;
  pl.splits = splits;
  pl.valid = true;
  L -= log2_int(splits);
  pl.slab_levels = L;
  const Variant& shallow = kVariants[tiling - 1][0];
  pl.deep = (L - 1) > shallow.levels_on_chip;
  const Variant& v = kVariants[tiling - 1][pl.deep ? 1 : 0];
  const int tile_m = v.pair ? 2 * BM : BM;
  pl.tiles_m = (M + tile_m - 1) / tile_m;
  pl.tiles_n = (N + v.bn - 1) / v.bn;
  const int num_tiles = pl.tiles_m * pl.tiles_n * splits;
  int ctas = sm_count(current_device());
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int units = v.pair ? ctas / 2 : ctas;
  if (units < 1) units = 1;
  if (units > num_tiles) units = num_tiles;
  pl.grid = v.pair ? 2 * units : units;
  pl.scratch_levels = (L - 1) > v.levels_on_chip ? (L - 1) - v.levels_on_chip : 0;
  pl.scratch_bytes = static_cast<size_t>(pl.grid) * pl.scratch_levels * v.level_bytes;
  // The head of every workspace belongs to the arrival counters, whether this launch uses them or not: a launch
  // that put its stack levels there would leave them non-zero for the next K-slab launch on the same workspace.
  pl.scratch_off = kCounterBytes;
  if (splits > 1) {
    // one arrival counter per 128-row block of an output tile
    if (static_cast<size_t>(pl.tiles_m) * pl.tiles_n * (v.pair ? 2 : 1) * sizeof(uint32_t) > kCounterBytes) pl.valid = false;
    pl.partial_off = (pl.scratch_off + pl.scratch_bytes + 255) & ~size_t(255);
    pl.partial_bytes = static_cast<size_t>(splits) * M * ((N + 7) / 8 * 8) * 2;
  }
  return pl;
}

// Rough time of a plan in microseconds, fitted to measurements under a CUDA graph with the weight streaming from
// HBM (N = 4096, K = 4096 and 12288, 1..256 rows of C, every tiling x 1..16 slabs): launch, prologue and pipeline
// fill cost 4 us; a CTA advances one 64-wide k-block every 0.155 us (32-column tile) .. 0.53 us (256 columns);
// all CTAs together cannot stream the operands faster than HBM delivers them (5.8 TB/s in this access pattern);
// with K-slabs the arrival protocol and the last CTA's pass over the roots add 2 - 5 us depending on the tiling.
static double plan_cost_us(const Plan& pl, int M, int N, int kblocks_total, int ctas) {
  const Variant& v = kVariants[pl.tiling - 1][pl.deep ? 1 : 0];
  const int items = pl.tiles_m * pl.tiles_n * pl.splits;
  const int units = v.pair ? ctas / 2 : ctas;
  const int waves = (items + units - 1) / (units > 0 ? units : 1);
  static const double per_kblock[6] = {0.223, 0.19, 0.53, 0.44, 0.171, 0.155};
  static const double slab_overhead[6] = {5.0, 5.0, 2.3, 4.0, 2.2, 5.0};
  const double stream_bytes = (static_cast<double>(N) + M) * kblocks_total * BK * 2;
  double stream = waves * static_cast<double>(kblocks_total / pl.splits) * per_kblock[pl.tiling - 1];
  if (stream < stream_bytes / 5.8e6) stream = stream_bytes / 5.8e6;
  double t = 4.0 + stream;
  if (pl.splits > 1)
    t += slab_overhead[pl.tiling - 1] + 0.3 * (log2_int(pl.splits) - 1) + static_cast<double>(pl.splits + 1) * M * N * 2 / 3.0e6;
  return t;
}

// Automatic choice: the first tiling, in order of measured speed at large M (256x128 per CTA pair: operands
// shared by two SMs, the whole tree stack in tensor memory, eight pipeline stages; then 128x256, 128x128),
// that still gives (nearly) every SM a tile.  128x256 needs the caller's scratch for the upper tree levels.
//
// With fewer rows of C than that (decode-sized M) the GEMM streams W from HBM and needs every SM pulling: every
// (tiling, slabs) combination that fits the caller's workspace is costed -- K cut into 1, 2, 4, 8 or 16 slabs, at
// most one wave of work items when K is cut -- and the cheapest wins.  `groups` is the number of level-0 groups of
// the tree (T / F), the finest cut that keeps every slab a whole subtree.  The choice is a function of the sizes
// only, and no choice changes a bit of the result.
static Plan auto_plan(int M, int N, int L, int groups, int kblocks_total, int max_ctas, size_t ws_bytes, bool have_ws) {
  int ctas = sm_count(current_device());
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int enough = ctas - ctas / 5;
  // Enough rows of C for every SM: one of the two CTA-pair tilings.  A 256x256 tile costs a little less than two
  // 256x128 tiles -- a third less operand traffic per flop, UMMAs twice as long; measured at M = 8192, leaf 256:
  // 1357 vs 1320 TFLOP/s at K = 4096, 1294 vs 1279 at K = 12288 -- and clearly less at short K, where the per-tile
  // costs (pipeline refill, storing C) weigh more (K = 512: 981 vs 752, K = 1536: 1251 vs 1077).  What decides
  // between them is the last, partial wave: whole waves of tiles x cost per tile.  The 256x256 tile needs the
  // caller's scratch for the tree levels above the second.
  const bool short_k = kblocks_total <= 24;
  {
    const int units = ctas / 2 > 0 ? ctas / 2 : 1;
    Plan cand[2] = {make_plan(2, M, N, L, max_ctas), make_plan(4, M, N, L, max_ctas)};
    double cost[2];
    bool usable[2];
    for (int i = 0; i < 2; ++i) {
      const int tiles = cand[i].tiles_m * cand[i].tiles_n;
      usable[i] = (cand[i].total_bytes() == 0 || (have_ws && cand[i].total_bytes() <= ws_bytes)) && 2 * tiles >= enough;
      cost[i] = static_cast<double>((tiles + units - 1) / units) * (i == 0 ? 1.0 : (short_k ? 1.7 : 1.94));
    }
    if (usable[0] && usable[1]) return cost[1] < cost[0] ? cand[1] : cand[0];
    if (usable[0]) return cand[0];
    if (usable[1]) return cand[1];
  }
  const int order[6] = {2, 4, 3, 1, 5, 6};
  constexpr int kOrder = 6;
  for (int i = 2; i < 4; ++i) {
    Plan pl = make_plan(order[i], M, N, L, max_ctas);
    if (pl.total_bytes() > 0 && !(have_ws && pl.total_bytes() <= ws_bytes)) continue;
    if (pl.tiles_m * pl.tiles_n >= enough) return pl;  // enough rows of C
  }
  Plan best{};
  double best_cost = 0.0;
  bool have = false;
  for (int i = 0; i < kOrder; ++i) {
    for (int s = 1; s <= kMaxSplits; s *= 2) {
      if (s > 1 && (!have_ws || s > groups)) break;
      Plan pl = make_plan(order[i], M, N, L, max_ctas, s);
      if (s > 1 && pl.tiles_m * pl.tiles_n * s * (kVariants[order[i] - 1][0].pair ? 2 : 1) > ctas) break;  // one wave only
      if (!pl.valid || (pl.total_bytes() > 0 && !(have_ws && pl.total_bytes() <= ws_bytes))) continue;
      const double c = plan_cost_us(pl, M, N, kblocks_total, ctas);
      if (!have || c < best_cost) {
        best = pl;
        best_cost = c;
        have = true;
      }
    }
  }
  if (!have) best = make_plan(1, M, N, L, max_ctas);
  return best;
}

// fp32 nodes: a stack level is BN fp32 columns of tensor memory, so a tiling carries (512 - 2 BN) / BN levels above
// level 0 (2 / 6 / 14 for 128- / 64- / 32-column tiles); no shared-memory or scratch levels, no K-slabs.
static int node32_levels(int bn) { return (static_cast<int>(TMEM_COLS) - 2 * bn) / bn; }

static Plan plan_node32(int tiling, int M, int N, int L, int max_ctas) {
  Plan pl{};
  const Variant& v = kVariants[tiling - 1][0];
  pl.tiling = tiling;
  pl.deep = false;
  pl.splits = 1;
  pl.slab_levels = L;
  pl.valid = (tiling == 1 || tiling == 2 || tiling == 5 || tiling == 6) && (L - 1) <= node32_levels(v.bn);
  const int tile_m = v.pair ? 2 * BM : BM;
  pl.tiles_m = (M + tile_m - 1) / tile_m;
  pl.tiles_n = (N + v.bn - 1) / v.bn;
  int ctas = sm_count(current_device());
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int units = v.pair ? ctas / 2 : ctas;
  if (units < 1) units = 1;
  if (units > pl.tiles_m * pl.tiles_n) units = pl.tiles_m * pl.tiles_n;
  pl.grid = v.pair ? 2 * units : units;
  pl.scratch_off = kCounterBytes;
  return pl;
}

// The first of the full-rate tilings (256x128 pair, 128x128) that gives (nearly) every SM a tile and can hold the
// tree; otherwise the tiling that can hold it and occupies the most SMs.
static Plan auto_plan_node32(int M, int N, int L, int max_ctas) {
  int ctas = sm_count(current_device());
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int enough = ctas - ctas / 5;
  const int order[4] = {2, 1, 5, 6};
  Plan best{};
  int best_ctas = -1;
  for (int i = 0; i < 4; ++i) {
    Plan pl = plan_node32(order[i], M, N, L, max_ctas);
    if (!pl.valid) continue;
    if (i < 2 && pl.grid >= enough) return pl;
    if (pl.grid > best_ctas) {
      best = pl;
      best_ctas = pl.grid;
    }
  }
  return best;  // .valid is false when no tiling can hold a tree this deep
}

size_t gemm_workspace_bytes(int M, int N, int64_t K, int leaf) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return 0;
  // what the automatic choice would like to have if scratch were unlimited
  return auto_plan(M, N, L, T / F, T * (leaf / BK), 0, ~size_t(0), true).total_bytes();
}

int gemm_plan_query(int M, int N, int64_t K, int leaf, int max_ctas, size_t ws_bytes, int out[4]) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return set_error(TBIK_ERR_SHAPE, "tbik_gemm_plan: bad sizes");
  const Plan pl = auto_plan(M, N, L, T / F, T * (leaf / BK), max_ctas, ws_bytes, ws_bytes > 0);
  out[0] = pl.tiling;
  out[1] = pl.splits;
  out[2] = pl.grid;
  out[3] = pl.deep ? 1 : 0;
  return TBIK_OK;
}

size_t gemm_split_workspace_bytes(int M, int N, int64_t K, int leaf, int tiling, int splits) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return 0;
  if (tiling < 1 || tiling > 6 || splits < 1 || splits > kMaxSplits || (splits & (splits - 1)) || splits > T / F) return 0;
  const Plan pl = make_plan(tiling, M, N, L, 0, splits);
  return pl.valid ? pl.total_bytes() : 0;
}

// `forced` (optional): a plan chosen by the caller (the entry point with built-in scratch picks one that fits it).
static int gemm_launch_plan(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                            int64_t ldc, int dtype, int leaf, int T, int F, const Plan& pl, void* workspace,
                            cudaStream_t stream, int node_dtype = TBIK_NODE_INPUT) {
  const Variant& v = kVariants[pl.tiling - 1][pl.deep ? 1 : 0];
  const int dev = current_device();

  // rows of A per TMA box: all 128 of a CTA's tile, or just enough for a decode-sized M (16, 32, 64)
  int a_box = BM;
  if (!v.pair && M <= 64) a_box = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, dtype, A, M, K, lda, a_box);
  if (rc != TBIK_OK) return rc;
  rc = make_tmap(&tb, dtype, W, N, K, ldw, v.pair ? v.bn / 2 : v.bn);
  if (rc != TBIK_OK) return rc;

  GemmParams p{};
  p.a_box_bytes = static_cast<uint32_t>(a_box) * BK * 2;
  p.C = C;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.kblocks_per_leaf = leaf / BK;
  p.T = T / pl.splits;
  p.F = F;
  p.L = pl.slab_levels;
  p.splits = pl.splits;
  p.split_stride = 0;
  p.tiles_m = pl.tiles_m;
  p.tiles_n = pl.tiles_n;
  p.group_m = v.pair ? 8 : 16;  // 2048 rows of A per group: a wave of CTAs covers a near-square block of C
  {
    // More rows than one group: ask L2 to keep the rows of A (evict last), which every wave of the group reads
    // again; W keeps the normal priority.  Measured at M = 8192 (o_proj / down_proj, TFLOP/s, burst and 1.5 s back
    // to back on one GPU): no hints 1250 / 1157 and 1038 / 996; A last + W normal 1263 / 1186 and 1063 / 1028; A last
    // + W first 1223 / 1151 and 1019 / 986; W first alone 1189 / 1128 and 992 / 969.
    // TBIK_GEMM_L2_HINTS = "ab" (two digits 0..2, for A and W) overrides the choice, for measurements.
    static const int forced = [] {
      const char* e = getenv("TBIK_GEMM_L2_HINTS");
      return (e && e[0] >= '0' && e[0] <= '2' && e[1] >= '0' && e[1] <= '2') ? (e[0] - '0') * 3 + (e[1] - '0') : -1;
    }();
    // On the 256x256 pair tile W does better with the same priority (one call, burst and 1.5 s back to back, o_proj /
    // down_proj: none 1319 / 1311 and 1127 / 1126; A last 1326 / 1315 and 1133 / 1130; both last 1336 / 1326 and 1140 / 1141).
    p.hint_a = M > 2048 ? 2 : 0;
    p.hint_b = (M > 2048 && v.pair && v.bn == 256) ? 2 : 0;
    if (forced >= 0) {
      p.hint_a = forced / 3;
      p.hint_b = forced % 3;
    }
  }
  p.scratch = workspace ? reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(workspace) + pl.scratch_off) : nullptr;
  p.scratch_levels = pl.scratch_levels;
  p.status = status_address(dev);

  // C through TMA stores when its layout allows a tensor map (64-column boxes of 128 rows); otherwise the
  // epilogue threads store their rows directly.
  CUtensorMap tc{};
  p.tma_store = 0;
  if (pl.splits > 1) {
    // slab roots go to the workspace with direct stores (pad columns up to a multiple of 8 included: they are
    // zeros, W has no such rows); the CTA that stores the last root of a tile adds the roots and writes C
    const int64_t ldp = (N + 7) / 8 * 8;
    p.out = C;
    p.ldo = ldc;
    p.n_out = N;
    p.C = static_cast<unsigned char*>(workspace) + pl.partial_off;
    p.ldc = ldp;
    p.N = static_cast<int>(ldp);
    p.split_stride = static_cast<int64_t>(M) * ldp;
    p.counters = static_cast<uint32_t*>(workspace);
  } else if (node_dtype != TBIK_NODE_FP32_OUT_FP32 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && ldc % 8 == 0 &&
             make_tmap(&tc, dtype, C, M, N, ldc, BM, true) == TBIK_OK) {
    p.tma_store = 1;
  }

  if (node_dtype == TBIK_NODE_FP32)
    return dtype == TBIK_DTYPE_BF16 ? launch_node32<__nv_bfloat16, false>(pl.tiling, ta, tb, tc, p, pl.grid, stream, dev)
                                    : launch_node32<__half, false>(pl.tiling, ta, tb, tc, p, pl.grid, stream, dev);
  if (node_dtype == TBIK_NODE_FP32_OUT_FP32)
    return dtype == TBIK_DTYPE_BF16 ? launch_node32<__nv_bfloat16, true>(pl.tiling, ta, tb, tc, p, pl.grid, stream, dev)
                                    : launch_node32<__half, true>(pl.tiling, ta, tb, tc, p, pl.grid, stream, dev);
  return dtype == TBIK_DTYPE_BF16 ? launch_variant<__nv_bfloat16>(pl.tiling, pl.deep, ta, tb, tc, p, pl.grid, stream, dev)
                                  : launch_variant<__half>(pl.tiling, pl.deep, ta, tb, tc, p, pl.grid, stream, dev);
}

static int gemm_check_args(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                           int64_t ldc, int dtype, int leaf, int node_dtype, int tiling, const void* workspace, int* T,
                           int* F, int* L) {
  if (dtype != TBIK_DTYPE_BF16 && dtype != TBIK_DTYPE_FP16)
    return set_error(TBIK_ERR_DTYPE, "tbik_gemm supports bf16 and fp16 operands");
  if (node_dtype != TBIK_NODE_INPUT && node_dtype != TBIK_NODE_FP32 && node_dtype != TBIK_NODE_FP32_OUT_FP32)
    return set_error(TBIK_ERR_DTYPE, "tbik_gemm: node_dtype must be TBIK_NODE_INPUT, TBIK_NODE_FP32 or TBIK_NODE_FP32_OUT_FP32");
  if (M < 0 || N < 0 || K <= 0) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: M, N must be >= 0 and K > 0");
  if (leaf <= 0 || leaf % BK != 0) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: leaf must be a positive multiple of 64");
  if (tiling < 0 || tiling > 6) return set_error(TBIK_ERR_ARG, "tbik_gemm: tiling must be 0..6");
  if (tree_shape(K, leaf, T, F, L) != TBIK_OK)
    return set_error(TBIK_ERR_SHAPE, "tbik_gemm: K must be a multiple of the leaf width");
  if (*L > 16) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: reduction tree deeper than 16 levels is not supported");
  if (M == 0 || N == 0) return TBIK_OK;
  if (!A || !W || !C) return set_error(TBIK_ERR_ARG, "tbik_gemm: null pointer");
  if (lda < K || ldw < K || ldc < N) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: leading dimension smaller than the row");
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) || (lda % 8) || (ldw % 8))
    return set_error(TBIK_ERR_ALIGN, "tbik_gemm: A and W must be 16-byte aligned with row strides that are multiples of 8 elements");
  if (reinterpret_cast<uintptr_t>(C) & (node_dtype == TBIK_NODE_FP32_OUT_FP32 ? 3u : 1u))
    return set_error(TBIK_ERR_ALIGN, "tbik_gemm: C must be aligned to its element size");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u))
    return set_error(TBIK_ERR_ALIGN, "tbik_gemm: workspace must be 16-byte aligned");
  return TBIK_OK;
}

int gemm_launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                int dtype, int leaf, int node_dtype, int max_ctas, int tiling, void* workspace, size_t ws_bytes,
                cudaStream_t stream, int splits) {
  int T, F, L;
  int rc = gemm_check_args(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, tiling, workspace, &T, &F, &L);
  if (rc != TBIK_OK || M == 0 || N == 0) return rc;
  const bool have_ws = workspace != nullptr && ws_bytes > 0;

  if (node_dtype != TBIK_NODE_INPUT) {
    // fp32 nodes: tensor-memory stack only, one work item per tile
    if (splits > 1) return set_error(TBIK_ERR_ARG, "tbik_gemm: K-slabs are not available with fp32 nodes");
    const Plan pl = tiling == 0 ? auto_plan_node32(M, N, L, max_ctas) : plan_node32(tiling, M, N, L, max_ctas);
    if (!pl.valid) {
      char msg[200];
      snprintf(msg, sizeof(msg),
               "tbik_gemm: with fp32 nodes a tree of %d levels does not fit tensor memory (at most 15 levels; 3 on the "
               "full-rate tilings): use a wider leaf", L);
      return set_error(TBIK_ERR_SHAPE, msg);
    }
    return gemm_launch_plan(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, T, F, pl, workspace, stream, node_dtype);
  }

  // splits: 0 = automatic (only together with tiling 0), 1 = none, else a power of two of whole subtrees
  if (splits < 0 || splits > kMaxSplits || (splits & (splits - 1)) != 0)
    return set_error(TBIK_ERR_ARG, "tbik_gemm: the number of K-slabs must be a power of two up to 16");
  if (splits > 1 && (tiling == 0 || splits > T / F))
    return set_error(TBIK_ERR_SHAPE, "tbik_gemm: K-slabs need an explicit tiling and at most T / F slabs (whole subtrees)");
  const Plan pl = tiling == 0 ? auto_plan(M, N, L, splits == 1 ? 1 : T / F, T * (leaf / BK), max_ctas, ws_bytes, have_ws)
                              : make_plan(tiling, M, N, L, max_ctas, splits > 1 ? splits : 1);
  if (!pl.valid) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: too many output tiles for K-slabs");
  if (pl.total_bytes() > 0 && (!have_ws || pl.total_bytes() > ws_bytes)) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "tbik_gemm: a reduction tree of %d levels needs %zu bytes of scratch for this tiling (got %zu); "
             "see tbik_gemm_workspace_bytes", L, pl.total_bytes(), have_ws ? ws_bytes : size_t(0));
    return set_error(TBIK_ERR_SHAPE, msg);
  }
  return gemm_launch_plan(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, T, F, pl, workspace, stream);
}

// ---------------------------------------------------------------- the entry point that allocates nothing
// Scratch for the upper stack levels, the K-slab roots and their arrival counters, built into the library image:
// every GPU that loads the library holds these bytes until the process exits.  32 MiB covers every schedule the
// automatic choice picks for a Qwen3-8B row-split layer (the K-slab roots of a decode-sized call are under
// 10 MiB) and the 128x256 tiling of its deepest tree (down_proj, 5 levels: 148 CTAs x 3 levels x 64 KiB =
// 27.75 MiB).  The array is zero when the module is loaded, which is the state the arrival counters need, and
// every call that completes leaves them zero again.
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t gemm_static_scratch_bytes() { return kStaticScratchBytes; }

// The schedule the automatic choice prefers, if its scratch fits the array; else the best one that fits --
// unless that would mean falling back from a full-rate tiling to the narrow decode tilings, which need no
// scratch at any size but would run a large problem several times slower without saying so.
static bool static_plan(int M, int N, int T, int F, int L, int leaf, Plan* out, size_t* want_bytes) {
  const Plan want = auto_plan(M, N, L, T / F, T * (leaf / BK), 0, ~size_t(0), true);
  *want_bytes = want.total_bytes();
  const Plan pl = want.total_bytes() <= kStaticScratchBytes
                      ? want
                      : auto_plan(M, N, L, T / F, T * (leaf / BK), 0, kStaticScratchBytes, true);
  const bool degraded = pl.tiling >= 5 && want.tiling < 5;
  if (!pl.valid || pl.total_bytes() > kStaticScratchBytes || degraded) return false;
  *out = pl;
  return true;
}

int gemm_static_accepts(int M, int N, int64_t K, int leaf) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK || L > 16) return 0;
  Plan pl{};
  size_t want = 0;
  return static_plan(M, N, T, F, L, leaf, &pl, &want) ? 1 : 0;
}

int gemm_launch_static(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                       int64_t ldc, int dtype, int leaf, int node_dtype, cudaStream_t stream) {
  // In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address
  // the kernel may use has to be asked for, once per device, with that device current.
  static std::atomic<void*> device_addr[kMaxDevices];
  // fp32 nodes keep their stack in tensor memory: no scratch of any kind, hence nothing to allocate either
  if (node_dtype == TBIK_NODE_FP32 || node_dtype == TBIK_NODE_FP32_OUT_FP32)
    return gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, 0, nullptr, 0, stream, 0);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return set_error(TBIK_ERR_ARG, "tbik_gemm_static: device index out of range");
  void* scratch = device_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    e = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (e != cudaSuccess || scratch == nullptr) return set_cuda_error(e, "cudaGetSymbolAddress(g_static_scratch)");
    device_addr[dev].store(scratch, std::memory_order_release);  // two racing first calls store the same address
  }
  int T, F, L;
  int rc = gemm_check_args(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, nullptr, &T, &F, &L);
  if (rc != TBIK_OK || M == 0 || N == 0) return rc;
  Plan pl{};
  size_t want_bytes = 0;
  if (!static_plan(M, N, T, F, L, leaf, &pl, &want_bytes)) {
    char msg[240];
    snprintf(msg, sizeof(msg),
             "tbik_gemm_static: these sizes need %zu bytes of scratch, more than the %zu bytes built into the "
             "library; use tbik_gemm_ws with a caller-owned buffer", want_bytes, kStaticScratchBytes);
    return set_error(TBIK_ERR_SHAPE, msg);
  }
  return gemm_launch_plan(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, T, F, pl, scratch, stream);
}

int gemm_status(uint32_t out[4]) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(uint32_t) * 4);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaMemcpyFromSymbol(g_gemm_status)");
  if (out[0] != 0) {
    uint32_t zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_gemm_status, zero, sizeof(zero));
  }
  return TBIK_OK;
}

}  // namespace tbik
