// Device-side pieces of the cross-GPU all-reduce kernels (the packed arithmetic is shared with the GEMM kernel,
// which adds K-slab roots with it): the flag layout inside each rank's IPC-mapped meta buffer, the
// peer-pointer record, bounded flag waits, the per-block epoch barrier and packed arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace tbik {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 320;  // up to two CTAs per SM

struct alignas(128) Signal {
  uint32_t epoch[kMaxBlocks][kMaxRanks];  // private to the owning rank: last epoch used by (block, thread)
  uint32_t flag[kMaxBlocks][kMaxRanks];   // written by peers: flag[b][r] = last epoch announced by rank r, block b
  // push schedule of the all-reduce: push_flag[b][r] is written by rank r's block b ("my reduced part of chunk c
  // of call k is in your scratch": (k << 12) + c + 1); push_calls[b] is private to the owning rank
  uint32_t push_flag[kMaxBlocks][kMaxRanks];
  uint32_t push_calls[kMaxBlocks];
};

struct alignas(16) RankData {
  const void* ptrs[kMaxRanks];
};

struct RankSignals {
  Signal* sig[kMaxRanks];
};

// status record (host-mapped): [0] code (0 ok, 1 barrier timeout) [1] rank [2] block [3] peer
//                              [4] expected epoch [5] seen value [6] which barrier (1 start, 2 middle, 3 end)
struct ArStatus {
  uint32_t w[8];
};

__device__ __forceinline__ uint64_t ar_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_flag_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_flag_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_pack(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Per-block barrier across `NG` ranks.  Returns false (for every thread of the block) if a wait
// ran out.  `which` only labels the status record.
template <int NG>
__device__ __forceinline__ bool block_barrier(const RankSignals& sg, Signal* self, int rank, ArStatus* status,
                                              uint64_t limit_ns, int which, uint32_t* smem_fail) {
  __syncthreads();  // all data accesses of the previous phase are done (and ordered before the release below)
  if (threadIdx.x < NG) {
    const int peer = threadIdx.x;
    const uint32_t e = self->epoch[blockIdx.x][peer] + 1u;
    self->epoch[blockIdx.x][peer] = e;
    st_flag_release(&sg.sig[peer]->flag[blockIdx.x][rank], e);
    const uint32_t* mine = &self->flag[blockIdx.x][peer];
    uint32_t seen = ld_flag_acquire(mine);
    if (static_cast<int32_t>(seen - e) < 0) {
      const uint64_t t0 = ar_timer_ns();
      uint32_t it = 0;
      while (true) {
        seen = ld_flag_acquire(mine);
        if (static_cast<int32_t>(seen - e) >= 0) break;
        if ((++it & 255u) == 0u && ar_timer_ns() - t0 > limit_ns) {
          if (atomicCAS(&status->w[0], 0u, 1u) == 0u) {
            status->w[1] = rank;
            status->w[2] = blockIdx.x;
            status->w[3] = peer;
            status->w[4] = e;
            status->w[5] = seen;
            status->w[6] = which;
            __threadfence_system();
          }
          *smem_fail = 1u;
          break;
        }
      }
    }
  }
  __syncthreads();
  return *smem_fail == 0u;
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  __device__ static uint4 add(uint4 a, uint4 b) {
    uint4 r;
    r.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x));
    r.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y));
    r.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z));
    r.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w));
    return r;
  }
  static constexpr int kPerPack = 4;
  __device__ static void up(uint4 a, float (&f)[8]) {
    f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
    f[4] = f[5] = f[6] = f[7] = 0.f;
  }
  __device__ static uint4 down(const float (&f)[8]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <>
struct Elem<__half> {
  __device__ static uint32_t add2(uint32_t a, uint32_t b) {
    __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static uint4 add(uint4 a, uint4 b) { return make_uint4(add2(a.x, b.x), add2(a.y, b.y), add2(a.z, b.z), add2(a.w, b.w)); }
  static constexpr int kPerPack = 8;
  __device__ static void up(uint4 a, float (&f)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 down(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Elem<__nv_bfloat16> {
  __device__ static uint32_t add2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static uint4 add(uint4 a, uint4 b) { return make_uint4(add2(a.x, b.x), add2(a.y, b.y), add2(a.z, b.z), add2(a.w, b.w)); }
  static constexpr int kPerPack = 8;
  __device__ static void up(uint4 a, float (&f)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  __device__ static uint4 down(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Bounded wait until *flag has reached `want` (wrap-safe).  On expiry a record goes to the status word.
__device__ __forceinline__ bool wait_flag_reached(const uint32_t* flag, uint32_t want, ArStatus* status, uint64_t limit_ns,
                                                  int rank, int peer, int which) {
  uint32_t seen = ld_flag_acquire(flag);
  if (static_cast<int32_t>(seen - want) >= 0) return true;
  const uint64_t t0 = ar_timer_ns();
  for (uint32_t it = 1;; ++it) {
    seen = ld_flag_acquire(flag);
    if (static_cast<int32_t>(seen - want) >= 0) return true;
    if ((it & 15u) == 0u) __nanosleep(64);
    if ((it & 255u) == 0u && ar_timer_ns() - t0 > limit_ns) {
      if (atomicCAS(&status->w[0], 0u, 1u) == 0u) {
        status->w[1] = rank;
        status->w[2] = blockIdx.x;
        status->w[3] = peer;
        status->w[4] = want;
        status->w[5] = seen;
        status->w[6] = which;
        __threadfence_system();
      }
      return false;
    }
  }
}

}  // namespace tbik
