// Cross-GPU all-reduce over CUDA-IPC mapped buffers (NVLink 5 / NVSwitch peer loads), no NCCL.
//
// tree mode   out[i] = ((x0+x1)+(x2+x3)) + ((x4+x5)+(x6+x7)), every add rounded to the element
//             type: the rank-pair tree that finishes the K-reduction tree of the row-split GEMM
//             (reference: custom_tree_all_reduce / packed_tree_reduce,
//              mini_allreduce/tbik_kernel/csrc/allreduce/custom_all_reduce.cuh:203-234, 301-312).
// linear mode out[i] = downcast(fp32(x0) + fp32(x1) + ... ) in rank order
//             (reference: cross_device_reduce_1stage / _2stage, same file :193-201, 236-299).
//
// Two schedules, same arithmetic per element so the bits do not depend on the schedule:
//   one-shot  every GPU loads all n buffers and reduces everything            (latency bound sizes)
//   two-shot  GPU r reduces the r-th 1/n of the packs into its scratch area, a fenced barrier,
//             then every GPU gathers the n reduced parts                      (bandwidth bound sizes)
//
//   push      two-shot whose second half does not pull: GPU r writes each reduced pack into its own result and
//             into every peer's scratch, so the reduce phase (inbound direction of the links) and the
//             distribution (outbound direction) run at the same time; a per-(block, source) flag tells the
//             peer which chunks have landed, and the peer copies them from its scratch into its result
//             locally                                                         (largest messages, n >= 4)
//
// Synchronisation is a per-block epoch barrier: block b of rank r stores its epoch into slot
// [b][r] of every peer's flag array and waits until each of its own slots has reached the epoch
// (wrap-safe signed compare, so one flag array serves consecutive barriers).  Every wait is
// bounded: when it runs out the kernel writes a record to a host-visible status word, skips the
// data phase and returns, so a missing peer can never hang the GPU.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <vector>

#include "ar_common.cuh"
#include "tbik_internal.h"

namespace tbik {

constexpr int kThreads = 512;
constexpr uint64_t kArWaitLimitNs = 2000000000ull;  // default bound of one barrier wait
constexpr size_t kPushMinBytesDefault = ~size_t(0);   // push schedule: only when configured

// A vector is VEC consecutive 16-byte packs moved by one load / store instruction (VEC = 2: 256-bit accesses).
template <int VEC>
struct Vec {
  uint4 q[VEC];
};

template <int VEC>
__device__ __forceinline__ Vec<VEC> ld_vec(const void* base, int64_t vidx) {
  Vec<VEC> v;
  if constexpr (VEC == 1) {
    v.q[0] = ld_pack(reinterpret_cast<const uint4*>(base) + vidx);
  } else {
    static_assert(VEC == 2, "vectors are 16 or 32 bytes");
    const void* p = reinterpret_cast<const char*>(base) + vidx * 32;
    asm volatile("ld.relaxed.sys.global.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.q[0].x), "=r"(v.q[0].y), "=r"(v.q[0].z), "=r"(v.q[0].w), "=r"(v.q[1].x), "=r"(v.q[1].y),
                   "=r"(v.q[1].z), "=r"(v.q[1].w)
                 : "l"(p)
                 : "memory");
  }
  return v;
}

template <int VEC>
__device__ __forceinline__ void st_vec(void* base, int64_t vidx, const Vec<VEC>& v) {
  if constexpr (VEC == 1) {
    reinterpret_cast<uint4*>(base)[vidx] = v.q[0];
  } else {
    void* p = reinterpret_cast<char*>(base) + vidx * 32;
    asm volatile("st.global.v8.u32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::"r"(v.q[0].x), "r"(v.q[0].y),
                 "r"(v.q[0].z), "r"(v.q[0].w), "r"(v.q[1].x), "r"(v.q[1].y), "r"(v.q[1].z), "r"(v.q[1].w), "l"(p)
                 : "memory");
  }
}

// NG vectors, one per rank, combined.  TREE: rank-pair tree in T; else rank order in fp32.
template <typename T, int NG, bool TREE, int VEC>
__device__ __forceinline__ Vec<VEC> combine(Vec<VEC> (&v)[NG]) {
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    if constexpr (TREE) {
#pragma unroll
      for (int stride = 1; stride < NG; stride *= 2) {
#pragma unroll
        for (int i = 0; i + stride < NG; i += 2 * stride) v[i].q[j] = Elem<T>::add(v[i].q[j], v[i + stride].q[j]);
      }
    } else {
      float acc[8], t[8];
      Elem<T>::up(v[0].q[j], acc);
#pragma unroll
      for (int r = 1; r < NG; ++r) {
        Elem<T>::up(v[r].q[j], t);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += t[i];
      }
      v[0].q[j] = Elem<T>::down(acc);
    }
  }
  return v[0];
}

// What every schedule's kernel gets.  Sizes are in vectors of VEC packs.
struct ArArgs {
  const RankData* dp;  // every rank's address of the registered buffer the message lives in
  RankSignals sg;
  Signal* self;
  void* out;
  int64_t nvec;     // length of the message
  int64_t in_off;   // where the message starts inside the registered buffer
  ArStatus* status;
  uint64_t limit_ns;
  uint64_t* trace;  // optional (host-mapped): [block][8] globaltimer stamps of the phases of the last launch
  int rank;
  int chunks;       // push schedule only
  int keep_input;   // one-shot: 1 = the caller promises not to overwrite the input before the NEXT collective of
                    // this communicator has passed its first barrier, so the closing barrier is left out
};

__device__ __forceinline__ void stamp(const ArArgs& a, int slot) {
  if (a.trace != nullptr && threadIdx.x == 0) a.trace[blockIdx.x * 8 + slot] = ar_timer_ns();
}

// Reduce vectors [lo, hi) of the message (indices relative to its start) and hand each result to `sink(i, v)`.
// UNROLL vectors per thread are in flight at once: all UNROLL * NG loads are issued before the first add.
template <typename T, int NG, bool TREE, int VEC, int UNROLL, typename Sink>
__device__ __forceinline__ void reduce_range(const RankData& dp, int64_t in_off, int64_t lo, int64_t hi, int64_t tid,
                                             int64_t stride, Sink sink) {
  int64_t idx = lo + tid;
  for (; idx + (UNROLL - 1) * stride < hi; idx += UNROLL * stride) {
    Vec<VEC> v[UNROLL][NG];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int r = 0; r < NG; ++r) v[u][r] = ld_vec<VEC>(dp.ptrs[r], in_off + idx + u * stride);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) sink(idx + u * stride, combine<T, NG, TREE, VEC>(v[u]));
  }
  for (; idx < hi; idx += stride) {
    Vec<VEC> v[NG];
#pragma unroll
    for (int r = 0; r < NG; ++r) v[r] = ld_vec<VEC>(dp.ptrs[r], in_off + idx);
    sink(idx, combine<T, NG, TREE, VEC>(v));
  }
}

// All-gather of the two-shot schedules: every rank's part of the result is fetched from that rank's scratch.  Same
// thread <-> same offset as in the reduce phase.  All NG loads of an offset (two offsets when the message is long
// enough) are in flight before the first store: a load answered over NVLink takes microseconds, and a thread that
// stored each vector before asking for the next one would move 16 bytes per round trip.
template <int NG, int VEC>
__device__ __forceinline__ void gather_parts(void* const (&scratch)[NG], void* out, int64_t part, int64_t last,
                                             int64_t tid, int64_t stride) {
  constexpr int GU = (NG >= 8 ? 2 : 4) / VEC;  // offsets per thread in flight: 16 packs of payload
  int64_t idx = tid;
  for (; idx + (GU - 1) * stride < part; idx += GU * stride) {
    Vec<VEC> v[GU][NG];
#pragma unroll
    for (int u = 0; u < GU; ++u) {
#pragma unroll
      for (int src = 0; src < NG; ++src) v[u][src] = ld_vec<VEC>(scratch[src], idx + u * stride);
    }
#pragma unroll
    for (int u = 0; u < GU; ++u) {
#pragma unroll
      for (int src = 0; src < NG; ++src) st_vec<VEC>(out, src * part + idx + u * stride, v[u][src]);
    }
  }
  for (; idx < last; idx += stride) {
    Vec<VEC> v[NG];
#pragma unroll
    for (int src = 0; src < NG; ++src)
      if (src == NG - 1 || idx < part) v[src] = ld_vec<VEC>(scratch[src], idx);
#pragma unroll
    for (int src = 0; src < NG; ++src)
      if (src == NG - 1 || idx < part) st_vec<VEC>(out, src * part + idx, v[src]);
  }
}

template <typename T, int NG, bool TREE, int VEC, int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) allreduce_oneshot_kernel(const ArArgs a) {
  __shared__ uint32_t fail;
  if (threadIdx.x == 0) fail = 0u;
  stamp(a, 0);
  const RankData dp = *a.dp;
  if (!block_barrier<NG>(a.sg, a.self, a.rank, a.status, a.limit_ns, 1, &fail)) return;
  stamp(a, 1);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  void* out = a.out;
  reduce_range<T, NG, TREE, VEC, UNROLL>(dp, a.in_off, 0, a.nvec, tid, stride,
                                         [&](int64_t i, const Vec<VEC>& v) { st_vec<VEC>(out, i, v); });
  stamp(a, 2);
  // peers may still be reading this rank's buffer: nobody leaves before everybody is done -- unless the caller
  // keeps the buffer untouched until a later collective's first barrier has said the same thing
  if (a.keep_input == 0) block_barrier<NG>(a.sg, a.self, a.rank, a.status, a.limit_ns, 3, &fail);
  stamp(a, 4);
}

template <typename T, int NG, bool TREE, int VEC, int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) allreduce_twoshot_kernel(const ArArgs a) {
  __shared__ uint32_t fail;
  if (threadIdx.x == 0) fail = 0u;
  stamp(a, 0);
  const RankData dp = *a.dp;
  const int rank = a.rank;
  const int64_t part = a.nvec / NG;
  const int64_t start = rank * part;
  const int64_t end = rank == NG - 1 ? a.nvec : start + part;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  void* scratch[NG];
#pragma unroll
  for (int r = 0; r < NG; ++r) scratch[r] = a.sg.sig[r] + 1;

  if (!block_barrier<NG>(a.sg, a.self, rank, a.status, a.limit_ns, 1, &fail)) return;
  stamp(a, 1);
  // reduce-scatter: this rank owns vectors [start, end)
  {
    void* mine = scratch[rank];
    reduce_range<T, NG, TREE, VEC, UNROLL>(dp, a.in_off, start, end, tid, stride,
                                           [&](int64_t i, const Vec<VEC>& v) { st_vec<VEC>(mine, i - start, v); });
  }
  stamp(a, 2);
  // release this rank's scratch writes / acquire the peers'
  if (!block_barrier<NG>(a.sg, a.self, rank, a.status, a.limit_ns, 2, &fail)) return;
  stamp(a, 3);
  // all-gather; `last` = length of the last rank's part (>= part)
  gather_parts<NG, VEC>(scratch, a.out, part, a.nvec - part * (NG - 1), tid, stride);
  stamp(a, 4);
}

// ---------------------------------------------------------------------------------------------------------------
// fp32 in, 16-bit out: the cross-rank levels of a tree whose nodes stay fp32.  Every rank contributes the fp32 root
// of its subtree; the rank-pair tree adds them in fp32; the sum is rounded ONCE to OutT.  A vector is 8 floats
// (one 256-bit load) and becomes one 16-byte pack of the result, so the two-shot schedule rounds in its reduce phase
// and gathers half the bytes.
template <typename OutT>
__device__ __forceinline__ uint4 round_pack(const Vec<2>& v) {
  float f[8];
  f[0] = __uint_as_float(v.q[0].x); f[1] = __uint_as_float(v.q[0].y);
  f[2] = __uint_as_float(v.q[0].z); f[3] = __uint_as_float(v.q[0].w);
  f[4] = __uint_as_float(v.q[1].x); f[5] = __uint_as_float(v.q[1].y);
  f[6] = __uint_as_float(v.q[1].z); f[7] = __uint_as_float(v.q[1].w);
  return Elem<OutT>::down(f);
}

template <typename OutT, int NG, int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) allreduce_cast_oneshot_kernel(const ArArgs a) {
  __shared__ uint32_t fail;
  if (threadIdx.x == 0) fail = 0u;
  stamp(a, 0);
  const RankData dp = *a.dp;
  if (!block_barrier<NG>(a.sg, a.self, a.rank, a.status, a.limit_ns, 1, &fail)) return;
  stamp(a, 1);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint4* out = reinterpret_cast<uint4*>(a.out);
  reduce_range<float, NG, true, 2, UNROLL>(dp, a.in_off, 0, a.nvec, tid, stride,
                                           [&](int64_t i, const Vec<2>& v) { out[i] = round_pack<OutT>(v); });
  stamp(a, 2);
  if (a.keep_input == 0) block_barrier<NG>(a.sg, a.self, a.rank, a.status, a.limit_ns, 3, &fail);
  stamp(a, 4);
}

template <typename OutT, int NG, int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) allreduce_cast_twoshot_kernel(const ArArgs a) {
  __shared__ uint32_t fail;
  if (threadIdx.x == 0) fail = 0u;
  stamp(a, 0);
  const RankData dp = *a.dp;
  const int rank = a.rank;
  const int64_t part = a.nvec / NG;
  const int64_t start = rank * part;
  const int64_t end = rank == NG - 1 ? a.nvec : start + part;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  void* scratch[NG];
#pragma unroll
  for (int r = 0; r < NG; ++r) scratch[r] = a.sg.sig[r] + 1;
  if (!block_barrier<NG>(a.sg, a.self, rank, a.status, a.limit_ns, 1, &fail)) return;
  stamp(a, 1);
  {
    uint4* mine = reinterpret_cast<uint4*>(scratch[rank]);
    reduce_range<float, NG, true, 2, UNROLL>(dp, a.in_off, start, end, tid, stride,
                                             [&](int64_t i, const Vec<2>& v) { mine[i - start] = round_pack<OutT>(v); });
  }
  stamp(a, 2);
  if (!block_barrier<NG>(a.sg, a.self, rank, a.status, a.limit_ns, 2, &fail)) return;
  stamp(a, 3);
  gather_parts<NG, 1>(scratch, a.out, part, a.nvec - part * (NG - 1), tid, stride);
  stamp(a, 4);
}

// Push schedule.  Every rank owns the r-th 1/n of the vectors, cut into `chunks` chunks; every block works on the
// same index set of every (chunk, part) on every rank, so block b of rank p only ever depends on block b of
// the other ranks.  No barrier after the first one: by the time a rank has seen all its flags, every peer has
// finished reading this rank's input and writing this rank's scratch.
template <typename T, int NG, bool TREE, int VEC, int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) allreduce_push_kernel(const ArArgs a) {
  __shared__ uint32_t fail;
  __shared__ uint32_t base_s;
  const int rank = a.rank;
  Signal* self = a.self;
  if (threadIdx.x == 0) {
    fail = 0u;
    // call counter kept on the device so that a captured graph advances it on every replay
    const uint32_t k = self->push_calls[blockIdx.x] + 1u;
    self->push_calls[blockIdx.x] = k;
    base_s = k << 12;
  }
  stamp(a, 0);
  const RankData dp = *a.dp;
  void* scratch[NG];
#pragma unroll
  for (int r = 0; r < NG; ++r) scratch[r] = a.sg.sig[r] + 1;
  // every rank has entered this call: inputs are final, nobody still reads last call's scratch
  if (!block_barrier<NG>(a.sg, self, rank, a.status, a.limit_ns, 1, &fail)) return;
  stamp(a, 1);
  const uint32_t base = base_s;
  const int chunks = a.chunks;
  const int64_t part = a.nvec / NG;
  const int64_t last_len = a.nvec - part * (NG - 1);
  const int64_t clen = (last_len + chunks - 1) / chunks;
  void* out = a.out;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t my_len = rank == NG - 1 ? last_len : part;
  const int64_t my_start = rank * part;

  auto reduce_chunk = [&](int c) {
    const int64_t lo = c * clen;
    int64_t hi = lo + clen;
    if (hi > my_len) hi = my_len;
    reduce_range<T, NG, TREE, VEC, UNROLL>(dp, a.in_off, my_start + lo, my_start + hi, tid, stride,
                                           [&](int64_t i, const Vec<VEC>& v) {
                                             st_vec<VEC>(out, i, v);
#pragma unroll
                                             for (int p = 0; p < NG; ++p)
                                               if (p != rank) st_vec<VEC>(scratch[p], i, v);
                                           });
    __syncthreads();  // the block's stores are ordered before the releases below
    if (threadIdx.x < NG && static_cast<int>(threadIdx.x) != rank)
      st_flag_release(&a.sg.sig[threadIdx.x]->push_flag[blockIdx.x][rank], base + static_cast<uint32_t>(c) + 1u);
  };
  auto gather_chunk = [&](int c) -> bool {
    if (threadIdx.x < NG && static_cast<int>(threadIdx.x) != rank) {
      if (!wait_flag_reached(&self->push_flag[blockIdx.x][threadIdx.x], base + static_cast<uint32_t>(c) + 1u, a.status,
                             a.limit_ns, rank, threadIdx.x, 4))
        fail = 1u;
    }
    __syncthreads();
    if (fail != 0u) return false;
    const int64_t lo = c * clen;
    // local copy scratch -> result; the loads of all sources are issued before the stores
    for (int64_t idx = lo + tid; idx < lo + clen; idx += stride) {
      Vec<VEC> v[NG];
#pragma unroll
      for (int src = 0; src < NG; ++src) {
        const int64_t len = src == NG - 1 ? last_len : part;
        if (src != rank && idx < len) v[src] = ld_vec<VEC>(scratch[rank], src * part + idx);
      }
#pragma unroll
      for (int src = 0; src < NG; ++src) {
        const int64_t len = src == NG - 1 ? last_len : part;
        if (src != rank && idx < len) st_vec<VEC>(out, src * part + idx, v[src]);
      }
    }
    return true;
  };
  for (int c = 0; c < chunks; ++c) {
    reduce_chunk(c);
    if (c >= 1 && !gather_chunk(c - 1)) return;
  }
  stamp(a, 2);
  gather_chunk(chunks - 1);
  stamp(a, 4);
}

// ==================================================================== host object
struct IpcKey {
  unsigned char b[sizeof(cudaIpcMemHandle_t)];
  bool operator<(const IpcKey& o) const { return memcmp(b, o.b, sizeof(b)) < 0; }
};

struct Communicator {
  int rank = 0, world = 0;
  bool full_nvlink = true;
  RankSignals sg{};
  Signal* self = nullptr;
  RankData* rd_next = nullptr;  // next free slot of the caller-owned device table
  RankData* rd_end = nullptr;
  std::unordered_map<const void*, RankData*> registered;
  std::vector<void*> graph_pending;  // inputs seen during stream capture, slots reserved in order
  std::map<IpcKey, char*> opened;
  size_t scratch_bytes = 8u << 20;
  size_t oneshot_max_bytes = 0;  // 0 = built-in policy
  int max_blocks = 0;            // 0 = built-in policy
  int threads = 0;               // 0 = built-in policy
  size_t push_min_bytes = 0;     // 0 = built-in policy
  int push_chunks = 0;           // 0 = built-in policy
  uint64_t wait_limit_ns = kArWaitLimitNs;
  ArStatus* status_host = nullptr;
  ArStatus* status_dev = nullptr;
  int sm_count = 0;
  bool poisoned = false;
  int vec_packs = 0;             // 0 / 1 = 128-bit accesses, 2 = 256-bit
  int loads_in_flight = 0;       // 0 = built-in policy
  int cluster_pairs = 1;         // launch CTAs as clusters of two (placement only)
  std::vector<cudaEvent_t> events;  // hand-overs between the two streams of the row-block pipeline
  uint64_t* trace_host = nullptr;  // phase stamps of the last launch (host-mapped), when tracing is on
  uint64_t* trace_dev = nullptr;
  int trace_blocks = 0;
};

static Communicator* as_comm(tbik_ar_t h) { return reinterpret_cast<Communicator*>(h); }

enum Schedule { kOneShot = 0, kTwoShot = 1, kPush = 2 };

// `pairs`: launch the CTAs as clusters of two.  The kernels use no cluster feature; the point is placement: a
// cluster occupies both SMs of a pair, so an all-reduce that runs beside a GEMM whose CTAs are themselves pairs
// takes whole pairs away from it instead of halves of many.
static int launch_fn(void (*kernel)(const ArArgs), const ArArgs& a, int blocks, int threads, cudaStream_t stream,
                     bool pairs) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pairs && blocks % 2 == 0) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a);
  if (e != cudaSuccess) return set_cuda_error(e, "all-reduce kernel launch");
  return TBIK_OK;
}

template <typename T, int NG, bool TREE, int VEC, int UNROLL>
static int launch_kernel(const ArArgs& a, int sched, int blocks, int threads, cudaStream_t stream, bool pairs) {
  void (*kernel)(const ArArgs) = allreduce_oneshot_kernel<T, NG, TREE, VEC, UNROLL>;
  if (sched == kPush) {
    if constexpr (NG >= 2) kernel = allreduce_push_kernel<T, NG, TREE, VEC, UNROLL>;
  } else if (sched == kTwoShot) {
    kernel = allreduce_twoshot_kernel<T, NG, TREE, VEC, UNROLL>;
  }
  return launch_fn(kernel, a, blocks, threads, stream, pairs);
}

// fp32 -> 16-bit variants: 16 packs of payload in flight per thread (8 for one and two ranks' worth of loads)
template <typename OutT>
static int launch_cast(int world, const ArArgs& a, int sched, int blocks, int threads, cudaStream_t stream, bool pairs) {
  void (*kernel)(const ArArgs) = nullptr;
  const bool two = sched == kTwoShot;
  switch (world) {
    case 1: kernel = allreduce_cast_oneshot_kernel<OutT, 1, 4>; break;
    case 2: kernel = two ? allreduce_cast_twoshot_kernel<OutT, 2, 4> : allreduce_cast_oneshot_kernel<OutT, 2, 4>; break;
    case 4: kernel = two ? allreduce_cast_twoshot_kernel<OutT, 4, 2> : allreduce_cast_oneshot_kernel<OutT, 4, 2>; break;
    case 8: kernel = two ? allreduce_cast_twoshot_kernel<OutT, 8, 1> : allreduce_cast_oneshot_kernel<OutT, 8, 1>; break;
    default: return set_error(TBIK_ERR_SHAPE, "tree all-reduce supports 1, 2, 4 or 8 ranks");
  }
  return launch_fn(kernel, a, blocks, threads, stream, pairs);
}

// `vec` = 16-byte packs per load instruction (1 or 2), `loads` = 16-byte packs a thread keeps in flight (0 = the
// built-in 16 for 4 and 8 ranks, 8 for 2).  The tuned variants exist for the path the row-split layer uses (bf16,
// tree order); everything else runs the built-in shape.
template <typename T, int NG, bool TREE>
static int launch_ar(const ArArgs& a, int sched, int blocks, int threads, cudaStream_t stream, int vec, int loads,
                     bool pairs) {
  constexpr int kDefaultUnroll = NG >= 6 ? 2 : 4;
  if constexpr (std::is_same<T, __nv_bfloat16>::value && TREE && NG >= 2) {
    int unroll = loads > 0 ? loads / (NG * vec) : kDefaultUnroll / vec;
    if (unroll < 1) unroll = 1;
    while (unroll * NG * vec > 32) unroll /= 2;  // at most 32 packs = 128 registers of payload per thread
    if (vec == 2) {
      switch (unroll) {
        case 1: return launch_kernel<T, NG, TREE, 2, 1>(a, sched, blocks, threads, stream, pairs);
        case 2: return launch_kernel<T, NG, TREE, 2, 2>(a, sched, blocks, threads, stream, pairs);
        case 4:
          if constexpr (NG <= 4) return launch_kernel<T, NG, TREE, 2, 4>(a, sched, blocks, threads, stream, pairs);
          break;
        case 8:
          if constexpr (NG <= 2) return launch_kernel<T, NG, TREE, 2, 8>(a, sched, blocks, threads, stream, pairs);
          break;
        default: break;
      }
      return launch_kernel<T, NG, TREE, 2, 1>(a, sched, blocks, threads, stream, pairs);
    }
    switch (unroll) {
      case 1: return launch_kernel<T, NG, TREE, 1, 1>(a, sched, blocks, threads, stream, pairs);
      case 2: return launch_kernel<T, NG, TREE, 1, 2>(a, sched, blocks, threads, stream, pairs);
      case 4: return launch_kernel<T, NG, TREE, 1, 4>(a, sched, blocks, threads, stream, pairs);
      case 8:
        if constexpr (NG <= 4) return launch_kernel<T, NG, TREE, 1, 8>(a, sched, blocks, threads, stream, pairs);
        break;
      case 16:
        if constexpr (NG <= 2) return launch_kernel<T, NG, TREE, 1, 16>(a, sched, blocks, threads, stream, pairs);
        break;
      default: break;
    }
  }
  return launch_kernel<T, NG, TREE, 1, kDefaultUnroll>(a, sched, blocks, threads, stream, pairs);
}

template <typename T, bool TREE>
static int dispatch_world(int world, const ArArgs& a, int sched, int blocks, int threads, cudaStream_t stream, int vec,
                          int loads, bool pairs) {
  switch (world) {
    case 1:
      if constexpr (TREE) return launch_ar<T, 1, TREE>(a, kOneShot, blocks, threads, stream, 1, 0, pairs);
      break;
    case 2: return launch_ar<T, 2, TREE>(a, sched, blocks, threads, stream, vec, loads, pairs);
    case 4: return launch_ar<T, 4, TREE>(a, sched, blocks, threads, stream, vec, loads, pairs);
    case 6:
      if constexpr (!TREE) return launch_ar<T, 6, TREE>(a, sched, blocks, threads, stream, vec, loads, pairs);
      break;
    case 8: return launch_ar<T, 8, TREE>(a, sched, blocks, threads, stream, vec, loads, pairs);
    default: break;
  }
  return set_error(TBIK_ERR_SHAPE, TREE ? "tree all-reduce supports 1, 2, 4 or 8 ranks"
                                        : "all-reduce supports 2, 4, 6 or 8 ranks");
}

// `inp`: the message.  With `reg_buffer` it is first copied there; with `reg_base` it is a byte range inside the
// registered buffer that starts at reg_base (a producer wrote it in place); else it must itself be registered
// (or the stream is capturing).
static int ar_run_impl(tbik_ar_t h, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer,
                       size_t reg_bytes, const void* reg_base, bool tree, cudaStream_t stream, int max_blocks = -1,
                       bool keep_input = false, int cast_dtype = -1) {
  Communicator* c = as_comm(h);
  if (!c) return set_error(TBIK_ERR_ARG, "all-reduce: null communicator");
  if (c->status_host && c->status_host->w[0] != 0) c->poisoned = true;
  if (c->poisoned)
    return set_error(TBIK_ERR_DEVICE, "all-reduce: an earlier call gave up waiting for a peer; the communicator must be rebuilt");
  const int esz = dtype == TBIK_DTYPE_FP32 ? 4 : 2;
  if (dtype != TBIK_DTYPE_FP32 && dtype != TBIK_DTYPE_FP16 && dtype != TBIK_DTYPE_BF16)
    return set_error(TBIK_ERR_DTYPE, "all-reduce supports float32, float16 and bfloat16");
  if (numel < 0) return set_error(TBIK_ERR_SHAPE, "all-reduce: negative element count");
  if (numel == 0) return TBIK_OK;
  if (!inp || !out) return set_error(TBIK_ERR_ARG, "all-reduce: null pointer");
  const size_t bytes = static_cast<size_t>(numel) * esz;
  if (bytes % 16 != 0)
    return set_error(TBIK_ERR_SHAPE, "all-reduce requires the byte size to be a multiple of 16");
  const bool cast = cast_dtype >= 0;
  if (cast) {
    // fp32 contributions, fp32 tree, one rounding to a 16-bit result: vectors of 8 elements
    if (dtype != TBIK_DTYPE_FP32 || !tree || (cast_dtype != TBIK_DTYPE_BF16 && cast_dtype != TBIK_DTYPE_FP16))
      return set_error(TBIK_ERR_DTYPE, "rounding all-reduce: float32 contributions, tree order, bfloat16 or float16 result");
    if (numel % 8 != 0) return set_error(TBIK_ERR_SHAPE, "rounding all-reduce: the element count must be a multiple of 8");
  }
  if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return set_error(TBIK_ERR_ALIGN, "all-reduce: out must be 16-byte aligned");

  const void* src = inp;
  if (reg_buffer) {
    if (bytes > reg_bytes) return set_error(TBIK_ERR_SHAPE, "all-reduce: input larger than the registered staging buffer");
    cudaError_t e = cudaMemcpyAsync(reg_buffer, inp, bytes, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaMemcpyAsync(staging)");
    src = reg_buffer;
  }
  if ((reinterpret_cast<uintptr_t>(src) & 15u) != 0) return set_error(TBIK_ERR_ALIGN, "all-reduce: input must be 16-byte aligned");
  size_t byte_off = 0;
  if (reg_base) {
    if (reinterpret_cast<uintptr_t>(src) < reinterpret_cast<uintptr_t>(reg_base))
      return set_error(TBIK_ERR_ARG, "all-reduce: the message lies before the registered buffer it was said to be in");
    byte_off = reinterpret_cast<uintptr_t>(src) - reinterpret_cast<uintptr_t>(reg_base);
    src = reg_base;
  }

  // Which slot of the device table describes this buffer on every rank?
  const RankData* slot = nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing(stream, &cap);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaStreamIsCapturing");
  auto it = c->registered.find(src);
  if (it != c->registered.end()) {
    slot = it->second;  // registered before: usable eagerly and under capture alike
  } else if (cap == cudaStreamCaptureStatusActive) {
    // Peer addresses are unknown until the handles are exchanged after capture: reserve the slot now.
    if (c->rd_next + c->graph_pending.size() + 1 > c->rd_end)
      return set_error(TBIK_ERR_STATE, "all-reduce: rank-data table is full");
    slot = c->rd_next + c->graph_pending.size();
    c->graph_pending.push_back(const_cast<void*>(src));
  } else {
    char msg[128];
    snprintf(msg, sizeof(msg), "buffer address %llu is not registered!", (unsigned long long)reinterpret_cast<uintptr_t>(src));
    return set_error(TBIK_ERR_STATE, msg);
  }

  const int64_t npacks = static_cast<int64_t>(bytes / 16);
  size_t one_max = c->oneshot_max_bytes;
  // two ranks: both schedules pull the same number of remote bytes, one-shot skips the scratch round trip
  // more ranks: measured on 8 GPUs, one-shot wins up to 1 MiB (26 vs 37 us at 512 KiB, 32 vs 38 us at 1 MiB), loses from 2 MiB
  if (one_max == 0) one_max = c->world <= 2 ? ~size_t(0) : (1u << 20);
  // rounding variant on two ranks: the two-shot schedule pulls 3/4 of the one-shot's bytes (half the fp32
  // contributions, then half the 16-bit result), which pays for its second barrier from 16 MiB of contributions on
  // (measured on 2 GPUs, one-shot / two-shot: 25.2 / 25.8 us at 4 MiB, 44.5 / 43.1 at 16, 121.7 / 97.9 at 64)
  if (cast && c->oneshot_max_bytes == 0 && c->world == 2) one_max = 8u << 20;
  bool twoshot = c->world > 1 && bytes > one_max && c->full_nvlink;
  if (twoshot) {
    // the last rank's part of the result in 16-byte packs, rounded up (rounding variant: 8 elements per pack)
    const int64_t part = (cast ? numel / 8 : npacks) / c->world + 2 * c->world;
    if (static_cast<size_t>(part) * 16 > c->scratch_bytes) {
      if (bytes <= (8u << 20)) twoshot = false;  // small enough for the one-shot schedule
      else return set_error(TBIK_ERR_SHAPE, "all-reduce: message needs more scratch than the meta buffer provides (raise max_size)");
    }
  }
  // push schedule: needs room for the whole message in every rank's scratch
  int push_chunks = 0;
  {
    const size_t push_min = c->push_min_bytes != 0 ? c->push_min_bytes : kPushMinBytesDefault;
    if (twoshot && bytes >= push_min && bytes <= c->scratch_bytes) {
      push_chunks = c->push_chunks > 0 ? c->push_chunks : 4;
      const int64_t part = npacks / (2 * c->world);
      if (push_chunks > part) push_chunks = part > 0 ? static_cast<int>(part) : 1;
    }
  }
  if (cast) {
    if (byte_off % 32 != 0 || (reinterpret_cast<uintptr_t>(src) & 31u) != 0)
      return set_error(TBIK_ERR_ALIGN, "rounding all-reduce: the contributions must be 32-byte aligned");
    push_chunks = 0;  // no push variant
  }
  // 256-bit accesses when asked for and every address involved is 32-byte aligned
  int vec = cast ? 2 : (c->vec_packs == 2 && dtype == TBIK_DTYPE_BF16 && tree && c->world >= 2) ? 2 : 1;
  if (vec == 2 && (npacks % 2 != 0 || byte_off % 32 != 0 || (reinterpret_cast<uintptr_t>(out) & 31u) != 0 ||
                   (reinterpret_cast<uintptr_t>(src) & 31u) != 0))
    vec = 1;
  const int64_t nvec = npacks / vec;
  const int64_t work = twoshot ? (nvec + c->world - 1) / c->world : nvec;
  const int want_blocks = max_blocks >= 0 ? max_blocks : c->max_blocks;
  int cap_blocks = want_blocks > 0 ? want_blocks : (bytes <= (256u << 10) ? 36 : c->sm_count);
  if (cap_blocks > kMaxBlocks) cap_blocks = kMaxBlocks;
  const int threads = c->threads > 0 ? c->threads : kThreads;
  // every block of a launch must be resident at once (block b waits for block b of the peers)
  const int resident = c->sm_count * (threads <= 256 ? 2 : 1);
  if (cap_blocks > resident) cap_blocks = resident;
  int blocks = static_cast<int>((work + threads - 1) / threads);
  if (blocks > cap_blocks) blocks = cap_blocks;
  if (blocks < 1) blocks = 1;

  ArArgs a{};
  a.dp = slot;
  a.sg = c->sg;
  a.self = c->self;
  a.out = out;
  a.nvec = nvec;
  a.in_off = static_cast<int64_t>(byte_off / (16 * vec));
  a.status = c->status_dev;
  a.limit_ns = c->wait_limit_ns;
  a.trace = c->trace_dev;
  a.rank = c->rank;
  a.chunks = push_chunks;
  a.keep_input = keep_input ? 1 : 0;
  if (c->trace_host) c->trace_blocks = blocks;
  const int sched = push_chunks > 0 ? kPush : (twoshot ? kTwoShot : kOneShot);
  const int loads = c->loads_in_flight;
  const bool pairs = c->cluster_pairs != 0 && blocks % 2 == 0;
  if (cast)
    return cast_dtype == TBIK_DTYPE_BF16 ? launch_cast<__nv_bfloat16>(c->world, a, sched, blocks, threads, stream, pairs)
                                         : launch_cast<__half>(c->world, a, sched, blocks, threads, stream, pairs);
  if (dtype == TBIK_DTYPE_FP32)
    return tree ? dispatch_world<float, true>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs)
                : dispatch_world<float, false>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs);
  if (dtype == TBIK_DTYPE_FP16)
    return tree ? dispatch_world<__half, true>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs)
                : dispatch_world<__half, false>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs);
  return tree ? dispatch_world<__nv_bfloat16, true>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs)
              : dispatch_world<__nv_bfloat16, false>(c->world, a, sched, blocks, threads, stream, vec, loads, pairs);
}

int ar_run(tbik_ar_t h, const void* inp, void* out, int64_t numel, int dtype, void* reg_buffer, size_t reg_bytes,
           bool tree, cudaStream_t stream) {
  return ar_run_impl(h, inp, out, numel, dtype, reg_buffer, reg_bytes, nullptr, tree, stream);
}

int ar_run_within(tbik_ar_t h, const void* reg_base, size_t byte_offset, void* out, int64_t numel, int dtype,
                  cudaStream_t stream) {
  if (!reg_base) return set_error(TBIK_ERR_ARG, "all-reduce: null registered buffer");
  return ar_run_impl(h, static_cast<const char*>(reg_base) + byte_offset, out, numel, dtype, nullptr, 0, reg_base, true,
                     stream);
}

int ar_run_rounding(tbik_ar_t h, const void* reg_base, size_t byte_offset, void* out, int64_t numel, int out_dtype,
                    cudaStream_t stream) {
  if (!reg_base) return set_error(TBIK_ERR_ARG, "all-reduce: null registered buffer");
  if (out_dtype != TBIK_DTYPE_BF16 && out_dtype != TBIK_DTYPE_FP16)
    return set_error(TBIK_ERR_DTYPE, "rounding all-reduce: the result is bfloat16 or float16");
  return ar_run_impl(h, static_cast<const char*>(reg_base) + byte_offset, out, numel, TBIK_DTYPE_FP32, nullptr, 0,
                     reg_base, true, stream, -1, false, out_dtype);
}

// Row-split layer as a pipeline over blocks of rows: the GEMM of block i + 1 runs on `main` while the tree
// all-reduce of block i runs on `side` with a few CTAs.  Everything is enqueued from here in one go (launches,
// event records and waits), so the host spends microseconds per block, not tens of them.
int ar_row_split_layer(tbik_ar_t h, const void* A, const void* W, void* out, int M, int N, int K, int64_t lda,
                       int64_t ldw, int dtype, int leaf, void* reg_base, size_t reg_bytes, void* workspace,
                       size_t ws_bytes, const int* block_rows, int nblk, int comm_ctas, cudaStream_t main,
                       cudaStream_t side) {
  Communicator* c = as_comm(h);
  if (!c) return set_error(TBIK_ERR_ARG, "row-split layer: null communicator");
  if (dtype != TBIK_DTYPE_BF16 && dtype != TBIK_DTYPE_FP16) return set_error(TBIK_ERR_DTYPE, "row-split layer: bf16 or fp16");
  if (M <= 0 || N <= 0 || K <= 0 || !A || !W || !out || !reg_base) return set_error(TBIK_ERR_ARG, "row-split layer: bad argument");
  if (static_cast<size_t>(M) * N * 2 > reg_bytes) return set_error(TBIK_ERR_SHAPE, "row-split layer: result larger than the registered buffer");
  if (N % 8 != 0) return set_error(TBIK_ERR_SHAPE, "row-split layer: N must be a multiple of 8");
  if (!block_rows || nblk < 1 || nblk > 64) return set_error(TBIK_ERR_ARG, "row-split layer: 1 to 64 blocks of rows");
  {
    int64_t total = 0;
    for (int b = 0; b < nblk; ++b) {
      if (block_rows[b] <= 0) return set_error(TBIK_ERR_SHAPE, "row-split layer: every block needs at least one row");
      total += block_rows[b];
    }
    if (total != M) return set_error(TBIK_ERR_SHAPE, "row-split layer: the blocks must add up to M rows");
  }
  if (main == side) return set_error(TBIK_ERR_ARG, "row-split layer: the two streams must differ");
  while (static_cast<int>(c->events.size()) < nblk + 1) {
    cudaEvent_t ev;
    cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaEventCreateWithFlags");
    c->events.push_back(ev);
  }
  if (comm_ctas < 2 || comm_ctas > c->sm_count / 2) return set_error(TBIK_ERR_ARG, "row-split layer: comm_ctas out of range");
  // (letting both kernels have every SM, the all-reduce as small CTAs beside the resident GEMM CTAs, was measured
  // too: it slows the GEMM more than the SMs given away here)
  const int gemm_ctas = c->sm_count - comm_ctas;
  const char* a = static_cast<const char*>(A);
  char* part = static_cast<char*>(reg_base);
  char* o = static_cast<char*>(out);
  int r0 = 0;
  for (int b = 0; b < nblk; r0 += block_rows[b], ++b) {
    const int rows = block_rows[b];
    const size_t off = static_cast<size_t>(r0) * N * 2;
    // the first block has the GPU to itself; the later ones leave SMs to the all-reduce of their predecessor
    int rc = gemm_launch(a + static_cast<size_t>(r0) * lda * 2, W, part + off, rows, N, K, lda, ldw, N, dtype, leaf,
                         TBIK_NODE_INPUT, b == 0 ? 0 : gemm_ctas, 0, workspace, ws_bytes, main, 0);
    if (rc != TBIK_OK) return rc;
    cudaError_t e = cudaEventRecord(c->events[b], main);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaEventRecord");
    e = cudaStreamWaitEvent(side, c->events[b], 0);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaStreamWaitEvent");
    const bool last = b == nblk - 1;
    // Only the layer's last all-reduce closes with a barrier: the blocks before it occupy other rows of the
    // registered buffer, which nobody writes again before that barrier has been passed.
    rc = ar_run_impl(h, part + off, o + off, static_cast<int64_t>(rows) * N, dtype, nullptr, 0, reg_base, true, side,
                     last ? 0 : comm_ctas, !last);
    if (rc != TBIK_OK) return rc;
  }
  cudaError_t e = cudaEventRecord(c->events[nblk], side);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaEventRecord");
  e = cudaStreamWaitEvent(main, c->events[nblk], 0);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaStreamWaitEvent");
  return TBIK_OK;
}

size_t ar_meta_size() { return sizeof(Signal); }

int ar_create(void* const* signals, int world, int rank, void* rank_data, size_t rank_data_bytes, int full_nvlink,
              tbik_ar_t* out) {
  if (!out || !signals) return set_error(TBIK_ERR_ARG, "tbik_ar_create: null pointer");
  if (world > kMaxRanks) return set_error(TBIK_ERR_SHAPE, "world size > 8 is not supported");
  if (world < 1 || (world != 1 && world % 2 != 0)) return set_error(TBIK_ERR_SHAPE, "Odd num gpus is not supported for now");
  if (rank < 0 || rank >= world) return set_error(TBIK_ERR_ARG, "invalid rank passed in");
  if (!rank_data || rank_data_bytes < sizeof(RankData)) return set_error(TBIK_ERR_ARG, "tbik_ar_create: rank_data table too small");
  for (int i = 0; i < world; ++i)
    if (!signals[i]) return set_error(TBIK_ERR_ARG, "tbik_ar_create: null signal pointer");
  Communicator* c = new Communicator();
  c->rank = rank;
  c->world = world;
  c->full_nvlink = full_nvlink != 0;
  for (int i = 0; i < world; ++i) c->sg.sig[i] = static_cast<Signal*>(signals[i]);
  c->self = c->sg.sig[rank];
  c->rd_next = static_cast<RankData*>(rank_data);
  c->rd_end = c->rd_next + rank_data_bytes / sizeof(RankData);
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (c->sm_count <= 0) c->sm_count = 1;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->status_host), sizeof(ArStatus), cudaHostAllocMapped);
  if (e != cudaSuccess) {
    delete c;
    return set_cuda_error(e, "cudaHostAlloc(status)");
  }
  memset(c->status_host, 0, sizeof(ArStatus));
  e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->status_dev), c->status_host, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(c->status_host);
    delete c;
    return set_cuda_error(e, "cudaHostGetDevicePointer(status)");
  }
  *out = c;
  return TBIK_OK;
}

int ar_destroy(tbik_ar_t h) {
  Communicator* c = as_comm(h);
  if (!c) return TBIK_OK;
  for (auto& kv : c->opened) cudaIpcCloseMemHandle(kv.second);
  if (c->status_host) cudaFreeHost(c->status_host);
  if (c->trace_host) cudaFreeHost(c->trace_host);
  for (cudaEvent_t ev : c->events) cudaEventDestroy(ev);
  delete c;
  return TBIK_OK;
}

int ar_configure(tbik_ar_t h, int key, int64_t value) {
  Communicator* c = as_comm(h);
  if (!c) return set_error(TBIK_ERR_ARG, "tbik_ar_configure: null communicator");
  switch (key) {
    case TBIK_AR_CFG_SCRATCH_BYTES: c->scratch_bytes = static_cast<size_t>(value); return TBIK_OK;
    case TBIK_AR_CFG_ONESHOT_MAX_BYTES: c->oneshot_max_bytes = static_cast<size_t>(value); return TBIK_OK;
    case TBIK_AR_CFG_MAX_BLOCKS: c->max_blocks = static_cast<int>(value); return TBIK_OK;
    case TBIK_AR_CFG_WAIT_LIMIT_NS: c->wait_limit_ns = static_cast<uint64_t>(value); return TBIK_OK;
    case TBIK_AR_CFG_PUSH_MIN_BYTES: c->push_min_bytes = static_cast<size_t>(value); return TBIK_OK;
    case TBIK_AR_CFG_PUSH_CHUNKS:
      if (value < 0 || value > 64) return set_error(TBIK_ERR_ARG, "tbik_ar_configure: push chunks must be 0..64");
      c->push_chunks = static_cast<int>(value);
      return TBIK_OK;
    case TBIK_AR_CFG_VEC_PACKS:
      if (value != 0 && value != 1 && value != 2) return set_error(TBIK_ERR_ARG, "tbik_ar_configure: vector width must be 0, 1 or 2 packs");
      c->vec_packs = static_cast<int>(value);
      return TBIK_OK;
    case TBIK_AR_CFG_LOADS_IN_FLIGHT:
      if (value < 0 || value > 32) return set_error(TBIK_ERR_ARG, "tbik_ar_configure: loads in flight must be 0..32");
      c->loads_in_flight = static_cast<int>(value);
      return TBIK_OK;
    case TBIK_AR_CFG_CLUSTER_PAIRS: c->cluster_pairs = value != 0 ? 1 : 0; return TBIK_OK;
    case TBIK_AR_CFG_TRACE:
      if (value != 0 && c->trace_host == nullptr) {
        cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&c->trace_host), sizeof(uint64_t) * 8 * kMaxBlocks, cudaHostAllocMapped);
        if (e != cudaSuccess) return set_cuda_error(e, "cudaHostAlloc(trace)");
        memset(c->trace_host, 0, sizeof(uint64_t) * 8 * kMaxBlocks);
        e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->trace_dev), c->trace_host, 0);
        if (e != cudaSuccess) return set_cuda_error(e, "cudaHostGetDevicePointer(trace)");
      } else if (value == 0 && c->trace_host != nullptr) {
        cudaFreeHost(c->trace_host);
        c->trace_host = c->trace_dev = nullptr;
      }
      return TBIK_OK;
    case TBIK_AR_CFG_THREADS:
      if (value != 0 && (value < 32 || value > kThreads || value % 32 != 0))
        return set_error(TBIK_ERR_ARG, "tbik_ar_configure: threads must be a multiple of 32 in [32, 512]");
      c->threads = static_cast<int>(value);
      return TBIK_OK;
    default: return set_error(TBIK_ERR_ARG, "tbik_ar_configure: unknown key");
  }
}

int ar_register_buffer(tbik_ar_t h, void* const* ptrs) {
  Communicator* c = as_comm(h);
  if (!c || !ptrs) return set_error(TBIK_ERR_ARG, "tbik_ar_register_buffer: null pointer");
  if (c->rd_next + c->graph_pending.size() + 1 > c->rd_end)
    return set_error(TBIK_ERR_STATE, "Rank data buffer is overflowed by 1");
  if (!c->graph_pending.empty())
    return set_error(TBIK_ERR_STATE, "tbik_ar_register_buffer: graph buffers are pending registration");
  RankData d{};
  for (int i = 0; i < c->world; ++i) d.ptrs[i] = ptrs[i];
  cudaError_t e = cudaMemcpy(c->rd_next, &d, sizeof(d), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaMemcpy(rank data)");
  c->registered[ptrs[c->rank]] = c->rd_next;
  ++c->rd_next;
  return TBIK_OK;
}

int ar_graph_meta_count(tbik_ar_t h, int* n) {
  Communicator* c = as_comm(h);
  if (!c || !n) return set_error(TBIK_ERR_ARG, "tbik_ar_graph_meta_count: null pointer");
  *n = static_cast<int>(c->graph_pending.size());
  return TBIK_OK;
}

int ar_graph_meta(tbik_ar_t h, void* handles_out, int64_t* offsets_out) {
  Communicator* c = as_comm(h);
  if (!c) return set_error(TBIK_ERR_ARG, "tbik_ar_graph_meta: null communicator");
  typedef CUresult (*GetAttrFn)(void*, CUpointer_attribute, CUdeviceptr);
  static GetAttrFn get_attr = nullptr;
  if (!get_attr && !c->graph_pending.empty()) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return set_error(TBIK_ERR_CUDA, "cuPointerGetAttribute is not available from the driver");
    get_attr = reinterpret_cast<GetAttrFn>(p);
  }
  for (size_t i = 0; i < c->graph_pending.size(); ++i) {
    void* ptr = c->graph_pending[i];
    void* base = nullptr;
    // the handle of an allocation always names its base address
    if (get_attr(&base, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
      return set_error(TBIK_ERR_CUDA, "failed to get pointer attr");
    cudaError_t e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(static_cast<char*>(handles_out) + i * sizeof(cudaIpcMemHandle_t)), base);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaIpcGetMemHandle");
    offsets_out[i] = static_cast<char*>(ptr) - static_cast<char*>(base);
  }
  return TBIK_OK;
}

int ar_register_graph_buffers(tbik_ar_t h, const void* const* handles, const int64_t* const* offsets) {
  Communicator* c = as_comm(h);
  if (!c || !handles || !offsets) return set_error(TBIK_ERR_ARG, "tbik_ar_register_graph_buffers: null pointer");
  const size_t n = c->graph_pending.size();
  if (c->rd_next + n > c->rd_end) return set_error(TBIK_ERR_STATE, "Rank data buffer is overflowed");
  if (n == 0) return TBIK_OK;
  std::vector<RankData> rd(n);
  for (size_t i = 0; i < n; ++i) {
    for (int j = 0; j < c->world; ++j) {
      if (j == c->rank) {
        rd[i].ptrs[j] = c->graph_pending[i];
        continue;
      }
      IpcKey key;
      memcpy(key.b, static_cast<const char*>(handles[j]) + i * sizeof(cudaIpcMemHandle_t), sizeof(key.b));
      auto it = c->opened.find(key);
      if (it == c->opened.end()) {
        void* p = nullptr;
        cudaIpcMemHandle_t hd;
        memcpy(&hd, key.b, sizeof(hd));
        cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return set_cuda_error(e, "cudaIpcOpenMemHandle");
        it = c->opened.emplace(key, static_cast<char*>(p)).first;
      }
      rd[i].ptrs[j] = it->second + offsets[j][i];
    }
  }
  cudaError_t e = cudaMemcpy(c->rd_next, rd.data(), sizeof(RankData) * n, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return set_cuda_error(e, "cudaMemcpy(graph rank data)");
  c->rd_next += n;
  c->graph_pending.clear();
  return TBIK_OK;
}

int ar_trace(tbik_ar_t h, uint64_t* out, int max_blocks, int* blocks) {
  Communicator* c = as_comm(h);
  if (!c || !out || !blocks) return set_error(TBIK_ERR_ARG, "tbik_ar_trace: null pointer");
  if (!c->trace_host) return set_error(TBIK_ERR_STATE, "tbik_ar_trace: tracing is off (TBIK_AR_CFG_TRACE)");
  const int n = c->trace_blocks < max_blocks ? c->trace_blocks : max_blocks;
  memcpy(out, c->trace_host, sizeof(uint64_t) * 8 * (n > 0 ? n : 0));
  *blocks = n;
  return TBIK_OK;
}

int ar_status(tbik_ar_t h, uint32_t out[8]) {
  Communicator* c = as_comm(h);
  if (!c || !out) return set_error(TBIK_ERR_ARG, "tbik_ar_status: null pointer");
  for (int i = 0; i < 8; ++i) out[i] = c->status_host ? c->status_host->w[i] : 0u;
  return TBIK_OK;
}

}  // namespace tbik
