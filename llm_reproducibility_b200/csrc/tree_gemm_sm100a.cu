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
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "ar_common.cuh"
#include "ptx_sm100a.cuh"
#include "tbik_internal.h"

namespace tbik {

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

// Fused GEMM + tree all-reduce: the last `comm_ctas` CTAs of the grid do not compute; they reduce and gather
// finished output tiles over peer memory while the other CTAs keep multiplying.
struct FusedDev {
  const RankData* rd;   // every rank's partial-result buffer ([M, N] row-major, IPC registered)
  RankSignals sg;       // every rank's flag area
  ArStatus* status;
  uint64_t limit_ns;
  int world, rank, comm_ctas;
  uint32_t epoch;
  void* out;            // this rank's final [M, N]
  int64_t ldo;
};

struct GemmParams {
  void* C;
  int64_t ldc;
  int M, N;
  int kblocks_per_leaf;  // leaf / 64
  int T, F, L;           // leaves per tile, level-0 radix, number of levels
  int tiles_m, tiles_n, group_m;  // tiles_m counts 128-row (single) or 256-row (pair) tiles
  uint32_t* scratch;     // global stack levels: [cta][level][chunk][word][epilogue thread]
  int scratch_levels;    // levels per CTA held in `scratch`
  FusedDev f;            // used by the FUSED instantiation only
  int tma_store;         // 1: write C with TMA stores staged in the shared-memory stack slot (tmap_c valid)
  int splits;            // K-slabs per output tile (power of two); slab s covers leaves [s*T, (s+1)*T) and writes
  int64_t split_stride;  // its subtree root to C + s * split_stride elements (C = the partial buffer when > 1)
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
  static constexpr uint32_t OFF_FULL = OFF_STACK + SLEVELS * LEVEL_WORDS * 4;
  static constexpr uint32_t OFF_EMPTY = OFF_FULL + 8 * STAGES;
  static constexpr uint32_t OFF_TFULL = OFF_EMPTY + 8 * STAGES;
  static constexpr uint32_t OFF_TEMPTY = OFF_TFULL + 16;
  static constexpr uint32_t OFF_EPI_BAR = OFF_TEMPTY + 16;   // rendezvous of the 8 epilogue warps
  static constexpr uint32_t OFF_TMEM_PTR = OFF_EPI_BAR + 8;
  static constexpr uint32_t OFF_ABORT = OFF_TMEM_PTR + 4;
  static constexpr uint32_t SMEM_BYTES = OFF_ABORT + 4 + 1024;   // + slack for the manual alignment
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

// ------------------------------------------------------------------ communication CTAs of the fused kernel
// Tile t is owned by rank t mod n.  The owner waits until every rank has published its partial tile,
// adds them in the rank-pair tree order ((0+1)+(2+3))+((4+5)+(6+7)) in the element type (the upper
// levels of the same reduction tree the GEMM started), writes the sum over its own partial tile and
// into its result, and publishes "done"; every other rank then copies the owner's tile into its own
// result.  Tiles are visited in the order the GEMM CTAs produce them, so the NVLink traffic of a tile
// overlaps the UMMAs of later tiles.
//
// Peer data is pulled with tiled TMA loads (one destination CTA, peer memory as the source) into two
// 64 KiB shared-memory buffers: the TMA unit keeps far more bytes in flight per SM than load
// instructions can, which is what NVLink latency needs.  A job is one box column-block of an owned tile
// (n loads, one per rank) or a whole tile to copy from its owner.  The next job is issued before the
// current one is consumed only if its flags are already up, so a communication CTA never blocks on
// another one while holding work that the other needs.  All waits are bounded; the final barrier keeps
// every rank's buffers untouched until all ranks have finished reading.
struct PeerMaps {
  CUtensorMap m[8];  // rank k's partial-result buffer, box = 64 columns x (128 or 64) rows
};

constexpr uint32_t COMM_BUF_BYTES = 65536;
constexpr int COMM_BUFS = 3;  // 192 KiB of loads in flight per communication CTA

template <typename T, int NG, int BN>
__device__ void comm_role_n(const GemmParams& p, const PeerMaps& maps, int cidx) {
  static_assert(BN == 256, "communication role is written for 128x256 tiles");
  constexpr int BOX_ROWS = NG == 8 ? 64 : 128;              // rows per 64-column box
  constexpr uint32_t BOXB = BOX_ROWS * 128;                   // bytes of one box
  constexpr int TILE_BOXES = (BM / BOX_ROWS) * (BN / 64);     // boxes of one tile (4 or 8), exactly one buffer
  constexpr int OWN_BOXES = COMM_BUF_BYTES / (NG * BOXB);     // boxes (per rank) one "reduce" job covers
  constexpr int OWN_JOBS = TILE_BOXES / OWN_BOXES;            // jobs per owned tile
  static_assert(TILE_BOXES * BOXB == COMM_BUF_BYTES && OWN_BOXES >= 1 && OWN_JOBS * OWN_BOXES == TILE_BOXES, "buffer plan");
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t fail;
  __shared__ uint32_t inflight_s;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + COMM_BUFS * COMM_BUF_BYTES;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(sgen + COMM_BUFS * COMM_BUF_BYTES + 64);
  const FusedDev& f = p.f;
  const int tid = threadIdx.x;
  if (tid == 0) {
    fail = 0u;
    inflight_s = 0u;
    *abort_flag = 0u;
    for (int i = 0; i < COMM_BUFS; ++i) mbar_init(bar0 + 8u * i, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const RankData rd = *f.rd;
  Signal* self = f.sg.sig[f.rank];
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int64_t row_packs = p.N / 8;  // 16-byte packs per row of the partial buffers
  const int64_t out_row_packs = f.ldo / 8;
  uint4* out = reinterpret_cast<uint4*>(f.out);
  uint4* mine = reinterpret_cast<uint4*>(const_cast<void*>(rd.ptrs[f.rank]));

  // job = (tile, sub): an owned tile is OWN_JOBS jobs, a tile to copy from its owner is one job
  auto owned = [&](int t) { return t % NG == f.rank; };
  auto advance = [&](int& t, int& sub) {
    if (owned(t) && sub + 1 < OWN_JOBS) {
      ++sub;
    } else {
      t += f.comm_ctas;
      sub = 0;
    }
  };
  auto box_xy = [&](int tm, int tn, int box, int& x, int& y) {
    x = tn * BN + (box % (BN / 64)) * 64;
    y = tm * BM + (box / (BN / 64)) * BOX_ROWS;
  };
  // thread 0: are the flags this job needs up?  block = wait for them (bounded)
  auto flags_up = [&](int t, int sub, bool block) -> bool {
    if (owned(t)) {
      if (sub != 0) return true;  // checked with the tile's first job
      for (int k = 0; k < NG; ++k) {
        const uint32_t* fl = &f.sg.sig[k]->tile_ready[t];
        if (block) {
          if (!wait_flag_reached(fl, f.epoch, f.status, f.limit_ns, f.rank, k, 5)) return false;
        } else if (static_cast<int32_t>(ld_flag_acquire(fl) - f.epoch) < 0) {
          return false;
        }
      }
      return true;
    }
    const int o = t % NG;
    const uint32_t* fl = &f.sg.sig[o]->tile_done[t];
    if (block) return wait_flag_reached(fl, f.epoch, f.status, f.limit_ns, f.rank, o, 6);
    return static_cast<int32_t>(ld_flag_acquire(fl) - f.epoch) >= 0;
  };
  // thread 0: start the TMA loads of a job into buffer `slot`
  auto issue = [&](int t, int sub, int slot) {
    int tm, tn, x, y;
    tile_coords(p, t, tm, tn);
    const uint32_t dst = sbase + slot * COMM_BUF_BYTES;
    const uint32_t bar = bar0 + 8u * slot;
    asm volatile("fence.proxy.async;" ::: "memory");  // flags were read by loads; the data is read by the TMA unit
    mbar_arrive_expect_tx(bar, COMM_BUF_BYTES);
    if (owned(t)) {
#pragma unroll
      for (int ob = 0; ob < OWN_BOXES; ++ob) {
        box_xy(tm, tn, sub * OWN_BOXES + ob, x, y);
#pragma unroll
        for (int k = 0; k < NG; ++k) tma_load_2d(dst + (ob * NG + k) * BOXB, &maps.m[k], x, y, bar);
      }
    } else {
#pragma unroll
      for (int bx = 0; bx < TILE_BOXES; ++bx) {
        box_xy(tm, tn, bx, x, y);
        tma_load_2d(dst + bx * BOXB, &maps.m[t % NG], x, y, bar);
      }
    }
  };

  int it = cidx, isub = 0, islot = 0;  // next job to issue (meaningful in thread 0)
  int ct = cidx, csub = 0, cslot = 0;  // next job to consume (all threads)
  uint32_t inflight = 0;               // thread 0's count of issued, not yet consumed jobs
  uint32_t phases = 0;                 // bit s = parity to wait for on buffer s
  while (true) {
    if (tid == 0) {
      // fill the ring; only block on flags when nothing is in flight, so that no communication CTA
      // ever holds back work another one is waiting for
      while (inflight < COMM_BUFS && it < num_tiles) {
        const bool block = inflight == 0;
        if (!flags_up(it, isub, block)) {
          if (block) fail = 1u;
          break;
        }
        issue(it, isub, islot);
        advance(it, isub);
        islot = islot + 1 == COMM_BUFS ? 0 : islot + 1;
        ++inflight;
      }
      inflight_s = inflight;
    }
    __syncthreads();
    if (fail != 0u || inflight_s == 0u) break;
    if (!mbar_wait_bounded(bar0 + 8u * cslot, (phases >> cslot) & 1u, abort_flag, f.limit_ns)) fail = 1u;
    phases ^= 1u << cslot;
    __syncthreads();
    if (fail != 0u) break;
    // ---- consume the job in buffer cslot
    int tm, tn;
    tile_coords(p, ct, tm, tn);
    const uint4* buf = reinterpret_cast<const uint4*>(sgen + cslot * COMM_BUF_BYTES);
    if (owned(ct)) {
      for (int i = tid; i < OWN_BOXES * BOX_ROWS * 8; i += blockDim.x) {
        const int ob = i / (BOX_ROWS * 8), j = i - ob * (BOX_ROWS * 8);
        uint4 v[NG];
#pragma unroll
        for (int k = 0; k < NG; ++k) v[k] = buf[(ob * NG + k) * (BOXB / 16) + j];
#pragma unroll
        for (int stride = 1; stride < NG; stride *= 2) {
#pragma unroll
          for (int k = 0; k + stride < NG; k += 2 * stride) v[k] = Elem<T>::add(v[k], v[k + stride]);
        }
        int x, y;
        box_xy(tm, tn, csub * OWN_BOXES + ob, x, y);
        const int r = y + (j >> 3);
        const int64_t c = x / 8 + (j & 7);
        if (r < p.M && c < row_packs) {
          mine[static_cast<int64_t>(r) * row_packs + c] = v[0];
          out[static_cast<int64_t>(r) * out_row_packs + c] = v[0];
        }
      }
    } else {
      for (int i = tid; i < TILE_BOXES * BOX_ROWS * 8; i += blockDim.x) {
        const int bx = i / (BOX_ROWS * 8), j = i - bx * (BOX_ROWS * 8);
        int x, y;
        box_xy(tm, tn, bx, x, y);
        const int r = y + (j >> 3);
        const int64_t c = x / 8 + (j & 7);
        if (r < p.M && c < row_packs) out[static_cast<int64_t>(r) * out_row_packs + c] = buf[i];
      }
    }
    __syncthreads();  // the buffer is free again; this rank's stores of the job are issued
    if (tid == 0) {
      if (owned(ct) && csub == OWN_JOBS - 1) {
        __threadfence_system();
        st_flag_release(&self->tile_done[ct], f.epoch);
      }
      --inflight;
    }
    advance(ct, csub);
    cslot = cslot + 1 == COMM_BUFS ? 0 : cslot + 1;
  }
  block_barrier<NG>(f.sg, self, f.rank, f.status, f.limit_ns, 7, &fail);
}

template <typename T, int BN>
__device__ void comm_role(const GemmParams& p, const PeerMaps& maps, int cidx) {
  if constexpr (BN == 256) {
    switch (p.f.world) {
      case 2: comm_role_n<T, 2, BN>(p, maps, cidx); break;
      case 4: comm_role_n<T, 4, BN>(p, maps, cidx); break;
      case 8: comm_role_n<T, 8, BN>(p, maps, cidx); break;
      default: break;
    }
  }
}

template <typename T, int BN, int STAGES, int SLEVELS, bool PAIR, bool FUSED = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tree_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const GemmParams p, const __grid_constant__ PeerMaps peers) {
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
  static_assert(!(FUSED && PAIR), "the fused variant is single-CTA");
  const int gemm_ctas = FUSED ? static_cast<int>(gridDim.x) - p.f.comm_ctas : static_cast<int>(gridDim.x);
  if constexpr (FUSED) {
    if (static_cast<int>(blockIdx.x) >= gemm_ctas) {
      comm_role<T, BN>(p, peers, static_cast<int>(blockIdx.x) - gemm_ctas);
      return;
    }
  }
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA)
    // elect.sync, not lane == 0: the compiler then knows that one thread runs the branch and feeds the TMA
    // and UMMA instructions from uniform registers directly, instead of looping over the active lanes
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      const int kblocks = p.T * p.kblocks_per_leaf;
      bool ok = true;
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
          mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, (kb0 + kb) * BK, row0, full_bar(stage));
          tma_load_2d(sa + A_STAGE_BYTES, &tmap_b, (kb0 + kb) * BK, wrow0, full_bar(stage));
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
          if (!mbar_wait_bounded(tempty_bar(a), aphase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            role_failed = 2;
            break;
          }
          tc_fence_after_sync();
          const uint32_t tmem_d = tmem_base + a * BN;
          // one 64-wide k-block: wait for its stage, four UMMAs, release the stage
          auto kblock = [&](int kb) -> bool {
            if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              ok = false;
              role_failed = 3;
              return false;
            }
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
          } else {
            for (int kb = 0; kb < p.kblocks_per_leaf; ++kb) {
              if (!kblock(kb)) break;
            }
          }
          if (ok) commit(tfull_bar(a));
        }
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------------------------------------ epilogue: drain + tree combine
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

    // C leaves through the TMA unit when possible: the finished tile is staged (128-byte swizzle) in the
    // shared-memory slot of stack level 1, which is free once the tree is complete, and one thread issues
    // one tiled store per 64 columns.  The slot may only be rewritten after those stores have read it.
    const bool tma_c = SLEVELS > 0 && p.tma_store != 0;
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
    int pending_tile = -1;  // fused: tile whose stores are in flight and whose "ready" flag is still to be raised
    auto publish_pending = [&]() {
      if constexpr (FUSED) {
        if (epi_tid == 0 && pending_tile >= 0) {
          bulk_wait_all();  // the tile's global writes are performed
          __threadfence_system();
          st_flag_release(&p.f.sg.sig[p.f.rank]->tile_ready[pending_tile], p.f.epoch);
          pending_tile = -1;
        }
      }
    };
    auto staging_release = [&]() {
      if (staging_busy) {
        if (epi_tid == 0) {
          if constexpr (FUSED) publish_pending(); else bulk_wait_read_all();
        }
        epi_sync();
        staging_busy = false;
      }
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
      }
    } else {
    uint32_t s0[NW];  // the open level-0 group; once it closes, the node that climbs the tree
    uint32_t leaf_ctr = 0;
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
        if (!mbar_wait_bounded(tfull_bar(a), aphase, abort_flag, WAIT_LIMIT_NS)) {
          ok = false;
          role_failed = 4;
          break;
        }
        tc_fence_after_sync();
        if constexpr (C_::TMEM_LEVELS > 0) tmem_wait_st();  // stack stores of earlier leaves have landed
        const uint32_t tacc = tmem_base + lane_off + a * BN + h * C_::COLS_PER_WARP;
        const bool add0 = c0 > 0;
        {
          // drain the accumulator chunk by chunk; the next chunk flies while this one is rounded and added
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
              s0[c * 16 + j] = add0 ? Pack16<T>::add(s0[c * 16 + j], v) : v;  // level 0: radix F, sequential
            }
          }
        }
        if (++c0 < p.F) continue;
        c0 = 0;
        // levels >= 1: binary counter over finished groups
        uint32_t gb = g++;
        int lvl = 1;
        while (lvl < p.L && (gb & 1u)) {
          uint32_t t[NW];
          stack_load(lvl, t);
#pragma unroll
          for (int w = 0; w < NW; ++w) s0[w] = Pack16<T>::add(t[w], s0[w]);
          gb >>= 1;
          ++lvl;
        }
        if (lvl < p.L) {
          if (lvl - 1 == C_::TMEM_LEVELS) staging_release();  // about to overwrite the staging slot
          stack_store(lvl, s0);
        } else if (tma_c) {
          staging_release();
          // the slot is laid out per thread as a stack level but per row as a staged tile: nobody may
          // write tile rows into it before every warp has popped its own level-1 words
          epi_sync();
          constexpr int CCH = C_::COLS_PER_WARP / 64;  // 64-column boxes per warp
          const int r = q * 32 + lane;
#pragma unroll
          for (int cc = 0; cc < CCH; ++cc) {
            uint8_t* box = reinterpret_cast<uint8_t*>(smem_stack) + (h * CCH + cc) * (BM * 128) + r * 128;
#pragma unroll
            for (int u = 0; u < 8; ++u)
              *reinterpret_cast<uint4*>(box + ((u ^ (r & 7)) << 4)) =
                  make_uint4(s0[cc * 32 + 4 * u], s0[cc * 32 + 4 * u + 1], s0[cc * 32 + 4 * u + 2], s0[cc * 32 + 4 * u + 3]);
          }
          fence_proxy_async_smem();
          epi_sync();
          if (ok && epi_tid == 0) {
            const uint32_t sbase = smem_base + C_::OFF_STACK;
            const int row0 = tm * TILE_M + static_cast<int>(cta_rank) * BM;
#pragma unroll
            for (int b = 0; b < BN / 64; ++b) tma_store_2d(&tmap_c, sbase + b * (BM * 128), tn * BN + b * 64, row0);
            bulk_commit_group();
            pending_tile = tile;
          }
          staging_busy = true;
        } else if (row < p.M) {
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
      }
    }
    publish_pending();
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

// ------------------------------------------------------------------ K-slab combine
// When a call has too few output tiles to give every SM one, K is cut into S slabs (S a power of two, each slab a
// whole subtree of the reduction tree), every (tile, slab) pair becomes a work item of the GEMM kernel above, and
// slab s writes its subtree root to part[s].  This kernel finishes the tree: out = the pairwise sum
// ((p0+p1)+(p2+p3))+... of the roots, every add rounded to the element type -- the same upper tree levels one CTA
// would have climbed, and the same arithmetic the rank-pair tree all-reduce applies to tensor-parallel shards.
constexpr int kMaxSplits = 16;

template <typename T, int S>
__global__ void __launch_bounds__(256)
slab_combine_kernel(const uint4* __restrict__ part, int64_t slab_packs, T* __restrict__ out, int M, int N, int64_t ldc,
                    int ldp_packs, bool vec_ok) {
  const int64_t total = static_cast<int64_t>(M) * ldp_packs;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint4 v[S];
#pragma unroll
    for (int k = 0; k < S; ++k) v[k] = part[k * slab_packs + i];
#pragma unroll
    for (int stride = 1; stride < S; stride *= 2) {
#pragma unroll
      for (int k = 0; k + stride < S; k += 2 * stride) v[k] = Elem<T>::add(v[k], v[k + stride]);
    }
    const int row = static_cast<int>(i / ldp_packs);
    const int col0 = static_cast<int>(i % ldp_packs) * 8;
    T* dst = out + static_cast<int64_t>(row) * ldc + col0;
    if (vec_ok && col0 + 8 <= N) {
      *reinterpret_cast<uint4*>(dst) = v[0];
    } else {
      const uint32_t w[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
      uint16_t* d16 = reinterpret_cast<uint16_t*>(dst);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (col0 + j < N) d16[j] = static_cast<uint16_t>(j & 1 ? w[j >> 1] >> 16 : w[j >> 1] & 0xFFFFu);
    }
  }
}

// ==================================================================== host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// Row-major [rows, K] 16-bit matrix, row stride `ld` elements, box = 64 (K) x `box_rows` rows.
int make_tmap(CUtensorMap* tm, int dtype, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows,
              bool quiet = false, bool swizzle = true) {
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
  return TBIK_OK;
}

__device__ uint32_t g_gemm_status[4];

template <typename T, int BN, int STAGES, int SLEVELS, bool PAIR, bool FUSED = false>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
           cudaStream_t stream, const PeerMaps* peers = nullptr) {
  static const PeerMaps no_peers{};
  const PeerMaps& pm = peers ? *peers : no_peers;
  using C_ = Cfg<BN, STAGES, SLEVELS, PAIR>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kernel = tree_gemm_kernel<T, BN, STAGES, SLEVELS, PAIR, FUSED>;
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(C_::SMEM_BYTES));
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(tree_gemm_kernel)");
    configured[dev] = true;
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, p, pm);
    if (e != cudaSuccess) return set_cuda_error(e, "tree_gemm_kernel launch");
  } else {
    kernel<<<grid, NUM_THREADS, C_::SMEM_BYTES, stream>>>(ta, tb, tc, p, pm);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_cuda_error(e, "tree_gemm_kernel launch");
  }
  return TBIK_OK;
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
                   const GemmParams& p, int grid, cudaStream_t stream) {
  switch (tiling) {
    case 1: return deep ? launch<T, 128, 4, 2, false>(ta, tb, tc, p, grid, stream) : launch<T, 128, 6, 0, false>(ta, tb, tc, p, grid, stream);
    case 2: return deep ? launch<T, 128, 5, 2, true>(ta, tb, tc, p, grid, stream) : launch<T, 128, 8, 0, true>(ta, tb, tc, p, grid, stream);
    case 3: return launch<T, 256, 3, 1, false>(ta, tb, tc, p, grid, stream);
    case 4: return launch<T, 256, 5, 1, true>(ta, tb, tc, p, grid, stream);
    case 5: return launch<T, 64, 8, 0, false>(ta, tb, tc, p, grid, stream);
    case 6: return launch<T, 32, 8, 0, false>(ta, tb, tc, p, grid, stream);
    default: return set_error(TBIK_ERR_ARG, "unknown tiling");
  }
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 1;
  }
  return cached[dev];
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
struct Plan {
  int tiling;  // 1..6
  bool deep;
  int grid;
  int tiles_m, tiles_n;
  int splits;             // K-slabs per output tile (1 = the whole tree in one CTA)
  int slab_levels;        // tree levels one work item climbs: L - log2(splits)
  int scratch_levels;
  size_t scratch_bytes;   // global stack levels
  size_t partial_off;     // offset of the slab roots in the workspace (0 when splits == 1)
  size_t partial_bytes;   // [splits][M][N rounded up to 8] elements
  size_t total_bytes() const { return splits > 1 ? partial_off + partial_bytes : scratch_bytes; }
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
  L -= log2_int(splits);
  pl.slab_levels = L;
  const Variant& shallow = kVariants[tiling - 1][0];
  pl.deep = (L - 1) > shallow.levels_on_chip;
  const Variant& v = kVariants[tiling - 1][pl.deep ? 1 : 0];
  const int tile_m = v.pair ? 2 * BM : BM;
  pl.tiles_m = (M + tile_m - 1) / tile_m;
  pl.tiles_n = (N + v.bn - 1) / v.bn;
  const int num_tiles = pl.tiles_m * pl.tiles_n * splits;
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int units = v.pair ? ctas / 2 : ctas;
  if (units < 1) units = 1;
  if (units > num_tiles) units = num_tiles;
  pl.grid = v.pair ? 2 * units : units;
  pl.scratch_levels = (L - 1) > v.levels_on_chip ? (L - 1) - v.levels_on_chip : 0;
  pl.scratch_bytes = static_cast<size_t>(pl.grid) * pl.scratch_levels * v.level_bytes;
  if (splits > 1) {
    pl.partial_off = (pl.scratch_bytes + 255) & ~size_t(255);
    pl.partial_bytes = static_cast<size_t>(splits) * M * ((N + 7) / 8 * 8) * 2;
  }
  return pl;
}

// Rough time of a plan in microseconds, fitted to measurements at 16..512 rows of C (N = 4096, K = 1536..12288):
// a CTA advances one 64-wide k-block every 0.155 us (32-column tile) .. 0.53 us (256 columns), launch and
// prologue cost 3.5 us, the combine kernel 2.5 us plus its bytes.  What counts is the k-blocks per CTA.
static double plan_cost_us(const Plan& pl, int M, int N, int kblocks_total, int ctas) {
  const Variant& v = kVariants[pl.tiling - 1][pl.deep ? 1 : 0];
  const int items = pl.tiles_m * pl.tiles_n * pl.splits;
  const int units = v.pair ? ctas / 2 : ctas;
  const int waves = (items + units - 1) / (units > 0 ? units : 1);
  const double per_kblock = v.bn >= 256 ? 0.53 : v.bn == 128 ? (v.pair ? 0.18 : 0.23) : v.bn == 64 ? 0.17 : 0.155;
  double t = 3.5 + waves * (kblocks_total / pl.splits) * per_kblock;
  if (pl.splits > 1) t += 2.5 + static_cast<double>(pl.splits + 1) * M * N * 2 / 3.0e6;  // combine launch + its bytes at 3 TB/s
  return t;
}

// Automatic choice: the first tiling, in order of measured speed at large M (256x128 per CTA pair: operands
// shared by two SMs, the whole tree stack in tensor memory, eight pipeline stages; then 128x256, 128x128),
// that still gives (nearly) every SM a tile; with few rows of C the GEMM streams W from HBM and needs all SMs
// pulling, so the narrow tilings follow.  128x256 needs the caller's scratch for the upper tree levels.
//
// When even the narrowest tiling leaves SMs idle (decode-sized M), K is cut into slabs as well: every candidate
// (tiling, slabs) that fits one wave and the caller's workspace is costed and the cheapest wins.  `groups` is the
// number of level-0 groups of the tree (T / F), the finest cut that keeps every slab a whole subtree.
static Plan auto_plan(int M, int N, int L, int groups, int kblocks_total, int max_ctas, size_t ws_bytes, bool have_ws) {
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int enough = ctas - ctas / 5;
  // short K (at most 6 leaves of 256): the per-tile costs (pipeline refill, storing C) weigh more than the
  // k-loop, and the 256x256 pair tile has half as many of them per flop (measured: K = 512 981 vs 752 TFLOP/s,
  // K = 1536 1251 vs 1077; from K = 2048 on the 256x128 pair tile wins)
  const bool short_k = kblocks_total <= 24;
  const int order[6] = {short_k ? 4 : 2, short_k ? 2 : 4, 3, 1, 5, 6};
  constexpr int kOrder = 6;
  Plan best{};
  bool have = false;
  for (int i = 0; i < kOrder; ++i) {
    if (!short_k && order[i] == 4) continue;  // long K: 256x256 only adds scratch need
    Plan pl = make_plan(order[i], M, N, L, max_ctas);
    if (pl.scratch_bytes > 0 && !(have_ws && pl.scratch_bytes <= ws_bytes)) continue;
    const Variant& pv = kVariants[order[i] - 1][pl.deep ? 1 : 0];
    if (pl.tiles_m * pl.tiles_n * (pv.pair ? 2 : 1) >= enough) {
      if (order[i] <= 4 || !have_ws || groups < 2) return pl;  // enough rows of C: no slabs
      best = pl;
      have = true;
      break;
    }
    if (!have || pl.tiles_m * pl.tiles_n > best.tiles_m * best.tiles_n) {
      best = pl;
      have = true;
    }
  }
  if (!have) best = make_plan(1, M, N, L, max_ctas);
  if (!have_ws || groups < 2) return best;
  double best_cost = plan_cost_us(best, M, N, kblocks_total, ctas);
  for (int i = 0; i < kOrder; ++i) {
    if (order[i] == 4) continue;
    for (int s = 2; s <= kMaxSplits && s <= groups; s *= 2) {
      Plan pl = make_plan(order[i], M, N, L, max_ctas, s);
      if (pl.tiles_m * pl.tiles_n * s * (kVariants[order[i] - 1][0].pair ? 2 : 1) > ctas) break;  // one wave only
      if (pl.total_bytes() > ws_bytes) continue;
      const double c = plan_cost_us(pl, M, N, kblocks_total, ctas);
      if (c < best_cost) {
        best = pl;
        best_cost = c;
      }
    }
  }
  return best;
}

size_t gemm_workspace_bytes(int M, int N, int64_t K, int leaf) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return 0;
  // what the automatic choice would like to have if scratch were unlimited
  return auto_plan(M, N, L, T / F, T * (leaf / BK), 0, ~size_t(0), true).total_bytes();
}

size_t gemm_split_workspace_bytes(int M, int N, int64_t K, int leaf, int tiling, int splits) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return 0;
  if (tiling < 1 || tiling > 6 || splits < 1 || splits > kMaxSplits || (splits & (splits - 1)) || splits > T / F) return 0;
  return make_plan(tiling, M, N, L, 0, splits).total_bytes();
}

template <typename T>
static int launch_combine(int splits, const void* part, T* out, int M, int N, int64_t ldc, cudaStream_t stream) {
  const int ldp_packs = (N + 7) / 8;
  const int64_t slab_packs = static_cast<int64_t>(M) * ldp_packs;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(out) & 15u) == 0 && ldc % 8 == 0;
  int64_t blocks = (slab_packs + 255) / 256;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const uint4* p4 = static_cast<const uint4*>(part);
  const int g = static_cast<int>(blocks);
  switch (splits) {
    case 2: slab_combine_kernel<T, 2><<<g, 256, 0, stream>>>(p4, slab_packs, out, M, N, ldc, ldp_packs, vec_ok); break;
    case 4: slab_combine_kernel<T, 4><<<g, 256, 0, stream>>>(p4, slab_packs, out, M, N, ldc, ldp_packs, vec_ok); break;
    case 8: slab_combine_kernel<T, 8><<<g, 256, 0, stream>>>(p4, slab_packs, out, M, N, ldc, ldp_packs, vec_ok); break;
    case 16: slab_combine_kernel<T, 16><<<g, 256, 0, stream>>>(p4, slab_packs, out, M, N, ldc, ldp_packs, vec_ok); break;
    default: return set_error(TBIK_ERR_ARG, "slab combine: unsupported slab count");
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "slab combine kernel launch");
  return TBIK_OK;
}

int gemm_launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                int dtype, int leaf, int node_dtype, int max_ctas, int tiling, void* workspace, size_t ws_bytes,
                cudaStream_t stream, int splits) {
  if (dtype != TBIK_DTYPE_BF16 && dtype != TBIK_DTYPE_FP16)
    return set_error(TBIK_ERR_DTYPE, "tbik_gemm supports bf16 and fp16 operands");
  if (node_dtype != TBIK_NODE_INPUT)
    return set_error(TBIK_ERR_DTYPE, "tbik_gemm: only node_dtype = TBIK_NODE_INPUT is implemented");
  if (M < 0 || N < 0 || K <= 0) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: M, N must be >= 0 and K > 0");
  if (leaf <= 0 || leaf % BK != 0) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: leaf must be a positive multiple of 64");
  if (tiling < 0 || tiling > 6) return set_error(TBIK_ERR_ARG, "tbik_gemm: tiling must be 0..6");
  int T, F, L;
  if (tree_shape(K, leaf, &T, &F, &L) != TBIK_OK)
    return set_error(TBIK_ERR_SHAPE, "tbik_gemm: K must be a multiple of the leaf width");
  if (L > 16) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: reduction tree deeper than 16 levels is not supported");
  if (M == 0 || N == 0) return TBIK_OK;
  if (!A || !W || !C) return set_error(TBIK_ERR_ARG, "tbik_gemm: null pointer");
  if (lda < K || ldw < K || ldc < N) return set_error(TBIK_ERR_SHAPE, "tbik_gemm: leading dimension smaller than the row");
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) || (lda % 8) || (ldw % 8))
    return set_error(TBIK_ERR_ALIGN, "tbik_gemm: A and W must be 16-byte aligned with row strides that are multiples of 8 elements");
  if (reinterpret_cast<uintptr_t>(C) & 1u) return set_error(TBIK_ERR_ALIGN, "tbik_gemm: C must be 2-byte aligned");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u))
    return set_error(TBIK_ERR_ALIGN, "tbik_gemm: workspace must be 16-byte aligned");
  const bool have_ws = workspace != nullptr && ws_bytes > 0;

  // splits: 0 = automatic (only together with tiling 0), 1 = none, else a power of two of whole subtrees
  if (splits < 0 || splits > kMaxSplits || (splits & (splits - 1)) != 0)
    return set_error(TBIK_ERR_ARG, "tbik_gemm: the number of K-slabs must be a power of two up to 16");
  if (splits > 1 && (tiling == 0 || splits > T / F))
    return set_error(TBIK_ERR_SHAPE, "tbik_gemm: K-slabs need an explicit tiling and at most T / F slabs (whole subtrees)");
  const Plan pl = tiling == 0 ? auto_plan(M, N, L, splits == 1 ? 1 : T / F, T * (leaf / BK), max_ctas, ws_bytes, have_ws)
                              : make_plan(tiling, M, N, L, max_ctas, splits > 1 ? splits : 1);
  if (pl.total_bytes() > 0 && (!have_ws || pl.total_bytes() > ws_bytes)) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "tbik_gemm: a reduction tree of %d levels needs %zu bytes of scratch for this tiling (got %zu); "
             "see tbik_gemm_workspace_bytes", L, pl.total_bytes(), have_ws ? ws_bytes : size_t(0));
    return set_error(TBIK_ERR_SHAPE, msg);
  }
  const Variant& v = kVariants[pl.tiling - 1][pl.deep ? 1 : 0];

  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, dtype, A, M, K, lda, BM);
  if (rc != TBIK_OK) return rc;
  rc = make_tmap(&tb, dtype, W, N, K, ldw, v.pair ? v.bn / 2 : v.bn);
  if (rc != TBIK_OK) return rc;

  GemmParams p{};
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
  p.scratch = static_cast<uint32_t*>(workspace);
  p.scratch_levels = pl.scratch_levels;
  void* status_ptr = nullptr;
  cudaGetSymbolAddress(&status_ptr, g_gemm_status);
  p.status = static_cast<uint32_t*>(status_ptr);

  // C through TMA stores when its layout allows a tensor map (64-column boxes of 128 rows); otherwise the
  // epilogue threads store their rows directly.
  CUtensorMap tc{};
  p.tma_store = 0;
  if (pl.splits > 1) {
    // slab roots go to the workspace with direct stores; the combine kernel writes C
    const int64_t ldp = (N + 7) / 8 * 8;
    p.C = static_cast<unsigned char*>(workspace) + pl.partial_off;
    p.ldc = ldp;
    p.split_stride = static_cast<int64_t>(M) * ldp;
  } else if ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && ldc % 8 == 0 &&
             make_tmap(&tc, dtype, C, M, N, ldc, BM, true) == TBIK_OK) {
    p.tma_store = 1;
  }

  rc = dtype == TBIK_DTYPE_BF16 ? launch_variant<__nv_bfloat16>(pl.tiling, pl.deep, ta, tb, tc, p, pl.grid, stream)
                                : launch_variant<__half>(pl.tiling, pl.deep, ta, tb, tc, p, pl.grid, stream);
  if (rc != TBIK_OK || pl.splits == 1) return rc;
  if (dtype == TBIK_DTYPE_BF16)
    return launch_combine<__nv_bfloat16>(pl.splits, p.C, static_cast<__nv_bfloat16*>(C), M, N, ldc, stream);
  return launch_combine<__half>(pl.splits, p.C, static_cast<__half*>(C), M, N, ldc, stream);
}

// ---------------------------------------------------------------- GEMM + tree all-reduce in one launch
int gemm_launch_fused(const void* A, const void* W, void* part, int M, int N, int K, int64_t lda, int64_t ldw, int dtype,
                      int leaf, void* workspace, size_t ws_bytes, const FusedArgs& fa, cudaStream_t stream) {
  if (dtype != TBIK_DTYPE_BF16 && dtype != TBIK_DTYPE_FP16)
    return set_error(TBIK_ERR_DTYPE, "fused GEMM + all-reduce supports bf16 and fp16");
  if (fa.world != 2 && fa.world != 4 && fa.world != 8)
    return set_error(TBIK_ERR_SHAPE, "fused GEMM + all-reduce supports 2, 4 or 8 ranks");
  if (M <= 0 || N <= 0 || K <= 0 || N % 8 != 0 || fa.ldo % 8 != 0 || fa.ldo < N)
    return set_error(TBIK_ERR_SHAPE, "fused GEMM + all-reduce: M, N, K > 0 and N, ldo multiples of 8");
  if (leaf <= 0 || leaf % BK != 0) return set_error(TBIK_ERR_SHAPE, "leaf must be a positive multiple of 64");
  int T, F, L;
  if (tree_shape(K, leaf, &T, &F, &L) != TBIK_OK || L > 16)
    return set_error(TBIK_ERR_SHAPE, "K must be a multiple of the leaf width (tree of at most 16 levels)");
  if (!A || !W || !part || !fa.out) return set_error(TBIK_ERR_ARG, "fused GEMM + all-reduce: null pointer");
  if (lda < K || ldw < K) return set_error(TBIK_ERR_SHAPE, "leading dimension smaller than the row");
  if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) || (lda % 8) || (ldw % 8) ||
      (reinterpret_cast<uintptr_t>(part) & 15u) || (reinterpret_cast<uintptr_t>(fa.out) & 15u) ||
      (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u)))
    return set_error(TBIK_ERR_ALIGN, "fused GEMM + all-reduce: operands must be 16-byte aligned, strides multiples of 8");
  const int sms = sm_count();
  int comm = fa.comm_ctas;
  if (comm < 2 || comm > sms / 2) return set_error(TBIK_ERR_ARG, "fused GEMM + all-reduce: comm_ctas out of range");
  const Plan pl = make_plan(3, M, N, L, sms - comm);
  if (pl.tiles_m * pl.tiles_n > kMaxTiles) return set_error(TBIK_ERR_SHAPE, "fused GEMM + all-reduce: too many output tiles");
  if (pl.scratch_bytes > 0 && (workspace == nullptr || pl.scratch_bytes > ws_bytes))
    return set_error(TBIK_ERR_SHAPE, "fused GEMM + all-reduce: scratch buffer too small for this tree");
  const Variant& v = kVariants[2][0];
  CUtensorMap ta, tb, tc;
  int rc = make_tmap(&ta, dtype, A, M, K, lda, BM);
  if (rc != TBIK_OK) return rc;
  rc = make_tmap(&tb, dtype, W, N, K, ldw, v.bn);
  if (rc != TBIK_OK) return rc;
  rc = make_tmap(&tc, dtype, part, M, N, N, BM);
  if (rc != TBIK_OK) return rc;
  GemmParams p{};
  p.C = part;
  p.ldc = N;
  p.M = M;
  p.N = N;
  p.kblocks_per_leaf = leaf / BK;
  p.T = T;
  p.F = F;
  p.L = L;
  p.tiles_m = pl.tiles_m;
  p.tiles_n = pl.tiles_n;
  p.group_m = 16;
  p.splits = 1;
  p.scratch = static_cast<uint32_t*>(workspace);
  p.scratch_levels = pl.scratch_levels;
  p.tma_store = 1;
  void* status_ptr = nullptr;
  cudaGetSymbolAddress(&status_ptr, g_gemm_status);
  p.status = static_cast<uint32_t*>(status_ptr);
  p.f.rd = static_cast<const RankData*>(fa.rank_data_slot);
  for (int i = 0; i < fa.world; ++i) p.f.sg.sig[i] = static_cast<Signal*>(fa.signals[i]);
  p.f.status = static_cast<ArStatus*>(fa.status_dev);
  p.f.limit_ns = fa.wait_limit_ns;
  p.f.world = fa.world;
  p.f.rank = fa.rank;
  p.f.comm_ctas = comm;
  p.f.epoch = fa.epoch;
  p.f.out = fa.out;
  p.f.ldo = fa.ldo;
  PeerMaps pm{};
  for (int k = 0; k < fa.world; ++k) {
    rc = make_tmap(&pm.m[k], dtype, fa.peer_parts[k], M, N, N, fa.world == 8 ? 64 : 128, false, /*swizzle=*/false);
    if (rc != TBIK_OK) return rc;
  }
  const int grid = pl.grid + comm;
  if (dtype == TBIK_DTYPE_BF16) return launch<__nv_bfloat16, 256, 3, 1, false, true>(ta, tb, tc, p, grid, stream, &pm);
  return launch<__half, 256, 3, 1, false, true>(ta, tb, tc, p, grid, stream, &pm);
}

size_t gemm_fused_workspace_bytes(int M, int N, int64_t K, int leaf) {
  int T, F, L;
  if (M <= 0 || N <= 0 || tree_shape(K, leaf, &T, &F, &L) != TBIK_OK) return 0;
  return make_plan(3, M, N, L, 0).scratch_bytes;
}

// ---------------------------------------------------------------- the entry point that allocates nothing
// Scratch for the upper stack levels, built into the library image: every GPU that loads the library
// holds these bytes until the process exits.  32 MiB covers every schedule the automatic choice picks
// for a Qwen3-8B row-split layer (the K-slab roots of a decode-sized call are under 10 MiB) and the
// 128x256 tiling of its deepest tree (down_proj, 5 levels: 148 CTAs x 3 levels x 64 KiB = 27.75 MiB).
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t gemm_static_scratch_bytes() { return kStaticScratchBytes; }

int gemm_launch_static(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw,
                       int64_t ldc, int dtype, int leaf, int node_dtype, cudaStream_t stream) {
  // In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address
  // the kernel may use has to be asked for, once per device, with that device current.
  static void* device_addr[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return set_error(TBIK_ERR_ARG, "tbik_gemm_static: device index out of range");
  if (device_addr[dev] == nullptr) {
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_static_scratch);
    if (e != cudaSuccess || addr == nullptr) return set_cuda_error(e, "cudaGetSymbolAddress(g_static_scratch)");
    device_addr[dev] = addr;
  }
  const size_t need = gemm_workspace_bytes(M, N, K, leaf);
  if (need > kStaticScratchBytes) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "tbik_gemm_static: these sizes need %zu bytes of scratch, more than the %zu bytes built into the "
             "library; use tbik_gemm_ws with a caller-owned buffer", need, kStaticScratchBytes);
    return set_error(TBIK_ERR_SHAPE, msg);
  }
  return gemm_launch(A, W, C, M, N, K, lda, ldw, ldc, dtype, leaf, node_dtype, 0, 0, device_addr[dev],
                     kStaticScratchBytes, stream, 0);
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
