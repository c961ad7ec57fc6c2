/* CPU oracle in plain C for the TP-invariant row-split path (TEST INFRASTRUCTURE ONLY).
 *
 * A second, independent restatement of the reference's reduction order, beside oracle/tbik_ref.py:
 * scalar loops, no library arithmetic, own 16-bit float conversions.  The tests hold it against the
 * stored outputs of the reference's own kernel and against the Python oracle; the product never
 * links or loads it.
 *
 * Reference lines restated:
 *   tree shape (T, F, L)          src/tbik/tree_based_matmul.py:240-249
 *   leaf dot in fp32, one rounding src/tbik/tree_based_matmul.py:121-140
 *   level 0 (radix F, left to right) and the binary carry chain above it
 *                                 src/tbik/tree_based_matmul.py:141-174
 *   rank-pair tree                src/tbik/tree_based_all_reduce.py:32-35,
 *                                 mini_allreduce/tbik_kernel/csrc/allreduce/custom_all_reduce.cuh:203-234
 *
 * The order of the fp32 additions INSIDE a leaf is left to the matrix unit in the reference (tl.dot);
 * here it is k = 0, 1, 2, ...  With integer-valued operands every order gives the same exact sum,
 * which is what the bit-exact tests use.
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -o oracle/libtbik_oracle.so oracle/tbik_ref.c   (oracle/build_c.py)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TBIK_ORACLE_BF16 0
#define TBIK_ORACLE_FP16 1

static float u32_as_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint32_t f32_as_u32(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

/* bfloat16: the upper half of an IEEE single; round to nearest, ties to even */
static float bf16_to_f32(uint16_t h) { return u32_as_f32((uint32_t)h << 16); }
static uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_as_u32(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN stays NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* IEEE half: 1 sign, 5 exponent, 10 mantissa bits */
static float fp16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return u32_as_f32(sign);
    /* subnormal: normalise */
    int e = -1;
    do {
      ++e;
      man <<= 1;
    } while ((man & 0x400u) == 0);
    man &= 0x3ffu;
    return u32_as_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
  }
  if (exp == 31) return u32_as_f32(sign | 0x7f800000u | (man << 13));
  return u32_as_f32(sign | ((exp + 112u) << 23) | (man << 13));
}
static uint16_t f32_to_fp16(float f) {
  const uint32_t u = f32_as_u32(f);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t abs = u & 0x7fffffffu;
  if (abs > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);  /* NaN */
  if (abs >= 0x477ff000u) {                                   /* rounds to >= 65520: infinity */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (abs < 0x33000001u) return sign;                         /* below half of the smallest subnormal */
  int32_t exp = (int32_t)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7fffffu) | 0x800000u;               /* 24 significant bits */
  int shift;                                                  /* bits to drop */
  int32_t hexp;
  if (exp < -14) {                                            /* subnormal half */
    shift = 13 + (-14 - exp);
    hexp = 0;
  } else {
    shift = 13;
    hexp = exp + 15;
  }
  uint32_t kept = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1u))) ++kept;
  uint32_t out;
  if (hexp == 0) {
    out = kept;                                               /* may carry into the exponent: still right */
  } else {
    out = ((uint32_t)hexp << 10) + (kept - 0x400u);          /* a mantissa carry bumps the exponent */
  }
  return (uint16_t)(sign | out);
}

static float up(uint16_t h, int dtype) { return dtype == TBIK_ORACLE_BF16 ? bf16_to_f32(h) : fp16_to_f32(h); }
static uint16_t down(float f, int dtype) { return dtype == TBIK_ORACLE_BF16 ? f32_to_bf16(f) : f32_to_fp16(f); }
/* a + b in the element type: the exact sum of two 16-bit floats fits fp32 or is decided far from a tie */
static uint16_t add16(uint16_t a, uint16_t b, int dtype) { return down(up(a, dtype) + up(b, dtype), dtype); }

/* conversions exposed so that the tests can hold them against another implementation */
void tbik_oracle_up(const uint16_t* in, float* out, int64_t n, int dtype) {
  for (int64_t i = 0; i < n; ++i) out[i] = up(in[i], dtype);
}
void tbik_oracle_down(const float* in, uint16_t* out, int64_t n, int dtype) {
  for (int64_t i = 0; i < n; ++i) out[i] = down(in[i], dtype);
}

int tbik_oracle_tree_shape(int64_t K, int leaf, int* T, int* F, int* L) {
  if (leaf <= 0 || K <= 0 || K % leaf != 0) return -2;
  int64_t t = K / leaf, f = t;
  int l = 1;
  while (f > 2 && f % 2 == 0) {
    f /= 2;
    ++l;
  }
  *T = (int)t;
  *F = (int)f;
  *L = l;
  return 0;
}

/* C[M,N] = A[M,K] * B[K,N], all row-major 16-bit floats, K reduced leaf by leaf in the tree order. */
int tbik_oracle_matmul(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K, int leaf, int dtype) {
  int T, F, L;
  if (dtype != TBIK_ORACLE_BF16 && dtype != TBIK_ORACLE_FP16) return -3;
  if (tbik_oracle_tree_shape(K, leaf, &T, &F, &L) != 0) return -2;
  int failed = 0;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);           /* fp32 accumulator of the current leaf */
    uint16_t* stack = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)N * (size_t)(L + 1));
    if (!acc || !stack) {
      failed = 1;
      free(acc);
      free(stack);
      continue;
    }
    uint16_t* s0 = stack;                                              /* open level-0 group */
    int c0 = 0;
    unsigned g = 0;
    for (int t = 0; t < T; ++t) {
      for (int n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int k = t * leaf; k < (t + 1) * leaf; ++k) {
        const float a = up(A[(size_t)m * K + k], dtype);
        const uint16_t* b = B + (size_t)k * N;
        for (int n = 0; n < N; ++n) acc[n] += a * up(b[n], dtype);
      }
      /* the leaf is rounded once, then joins the open level-0 group (sequential sum of F leaves) */
      for (int n = 0; n < N; ++n) {
        const uint16_t v = down(acc[n], dtype);
        s0[n] = c0 > 0 ? add16(s0[n], v, dtype) : v;
      }
      if (++c0 < F) continue;
      c0 = 0;
      /* binary counter over finished groups: a set bit at level l means a pending left operand there */
      unsigned gb = g++;
      int lvl = 1;
      while (lvl < L && (gb & 1u)) {
        uint16_t* left = stack + (size_t)lvl * N;
        for (int n = 0; n < N; ++n) s0[n] = add16(left[n], s0[n], dtype);
        gb >>= 1;
        ++lvl;
      }
      if (lvl < L) {
        memcpy(stack + (size_t)lvl * N, s0, sizeof(uint16_t) * (size_t)N);
      } else {
        memcpy(C + (size_t)m * N, s0, sizeof(uint16_t) * (size_t)N);
      }
    }
    free(acc);
    free(stack);
  }
  return failed ? -5 : 0;
}

/* The same tree with fp32 nodes (the CUDA library's fp32-node mode; the reference has no such mode): a leaf is the
 * fp32 dot as it stands, every node is one fp32 add, nothing is rounded.  C32[M,N] receives the unrounded root; the
 * caller rounds it once (tbik_oracle_down) when it wants a 16-bit result. */
int tbik_oracle_matmul_fp32_nodes(const uint16_t* A, const uint16_t* B, float* C32, int M, int N, int K, int leaf,
                                  int dtype) {
  int T, F, L;
  if (dtype != TBIK_ORACLE_BF16 && dtype != TBIK_ORACLE_FP16) return -3;
  if (tbik_oracle_tree_shape(K, leaf, &T, &F, &L) != 0) return -2;
  int failed = 0;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
    float* stack = (float*)malloc(sizeof(float) * (size_t)N * (size_t)(L + 1));
    if (!acc || !stack) {
      failed = 1;
      free(acc);
      free(stack);
      continue;
    }
    float* s0 = stack;
    int c0 = 0;
    unsigned g = 0;
    for (int t = 0; t < T; ++t) {
      for (int n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int k = t * leaf; k < (t + 1) * leaf; ++k) {
        const float a = up(A[(size_t)m * K + k], dtype);
        const uint16_t* b = B + (size_t)k * N;
        for (int n = 0; n < N; ++n) acc[n] += a * up(b[n], dtype);
      }
      for (int n = 0; n < N; ++n) s0[n] = c0 > 0 ? s0[n] + acc[n] : acc[n];
      if (++c0 < F) continue;
      c0 = 0;
      unsigned gb = g++;
      int lvl = 1;
      while (lvl < L && (gb & 1u)) {
        const float* left = stack + (size_t)lvl * N;
        for (int n = 0; n < N; ++n) s0[n] = left[n] + s0[n];
        gb >>= 1;
        ++lvl;
      }
      memcpy(lvl < L ? stack + (size_t)lvl * N : C32 + (size_t)m * N, s0, sizeof(float) * (size_t)N);
    }
    free(acc);
    free(stack);
  }
  return failed ? -5 : 0;
}

/* out = ((p0 + p1) + (p2 + p3)) + ((p4 + p5) + (p6 + p7)), every add in the element type. */
int tbik_oracle_tree_allreduce(const uint16_t* const* parts, int world, uint16_t* out, int64_t numel, int dtype) {
  if (world < 1 || world > 8 || (world & (world - 1)) != 0) return -2;
  if (dtype != TBIK_ORACLE_BF16 && dtype != TBIK_ORACLE_FP16) return -3;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < numel; ++i) {
    uint16_t v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) v[r] = parts[r][i];
    for (int stride = 1; stride < world; stride *= 2)
      for (int k = 0; k + stride < world; k += 2 * stride) v[k] = add16(v[k], v[k + stride], dtype);
    out[i] = v[0];
  }
  return 0;
}
