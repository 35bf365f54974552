// Shared host/device helpers for the gridbook_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/gridbook_b200.h"

#define GB_DEVINL __device__ __forceinline__

// ---------------------------------------------------------------------------
// host-side error plumbing
// ---------------------------------------------------------------------------
void gb_set_error(const char* fmt, ...);
int gb_fail(int code, const char* fmt, ...);
int gb_sm_count();                 // SMs of the current device (cached)
int* gb_status_word();             // device int the kernels raise on a timed-out wait

bool gb_pdl_enabled();             // false when GRIDBOOK_B200_PDL=0 (plain stream order)
void gb_count_launch();            // every kernel launch of this library bumps gb_launch_count()

// Kernel launch with the programmatic-stream-serialization attribute (see gb_pdl_wait).
template <typename... KArgs, typename... Args>
inline cudaError_t gb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = gb_pdl_enabled() ? 1 : 0;
  gb_count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define GB_REQUIRE(cond, ...)                           \
  do {                                                  \
    if (!(cond)) return gb_fail(GB_EINVAL, __VA_ARGS__); \
  } while (0)

#define GB_CUDA_OK(expr)                                                       \
  do {                                                                         \
    cudaError_t e_ = (expr);                                                   \
    if (e_ != cudaSuccess)                                                     \
      return gb_fail(GB_ECUDA, "%s: %s", #expr, cudaGetErrorString(e_));       \
  } while (0)

#define GB_LAUNCH_OK(name)                                                     \
  do {                                                                         \
    cudaError_t e_ = cudaGetLastError();                                       \
    if (e_ != cudaSuccess)                                                     \
      return gb_fail(GB_ECUDA, "launch of %s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

int gb_check_format(const gb_format& f, int64_t K);
int gb_check_weight(const gb_weight* w);
int gb_prepare_kernels();          // per-device function attributes of the big kernels
int gb_prepare_gemm();
int gb_prepare_dot();
int gb_prepare_umma();
int gb_prepare_tab();
int gb_prepare_gemm_fp4();
// Longest a device-side wait may spin before it gives up and raises the status word
// (two seconds unless gb_set_wait_limit_ms changed it).
unsigned long long gb_wait_limit_ns();
// Swizzled (128-byte) operand map over a row-major [rows, K] matrix of 2- or 1-byte elements:
// box = 128 bytes of K x box_rows rows, rows past the end read zero.
int gb_tensor_map_operand(void* map_out, const void* base, int64_t rows, int64_t K, int elem_bytes, int box_rows);
// 1..128 activation rows of the literal format, the two-tier k = 16 format with 80-byte superblocks
// or the fp8 k = 32 format: decode into tensor memory, tcgen05 MMA with the weights on the M side
// (gb_gemv_umma.cu); GB_EUNSUPPORTED when the format, layout or row count is not its own.
int gb_gemv_umma(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                 int64_t workspace_bytes, void* stream);
int64_t gb_gemv_umma_workspace_bytes(int64_t M, int64_t N, int64_t K);
int gb_gemv_umma_max_rows(const gb_weight* w);
bool gb_gemv_umma_is_literal(const gb_weight* w);
int gb_tensor_map_bytes_2d(void* map_out, const void* base, uint64_t inner_bytes, uint64_t rows,
                           uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows);
// M = 1 literal-format linear by per-column inner-product tables (gb_gemv_dot.cu); GB_EUNSUPPORTED when
// the shape or layout is not its own, and the caller falls back to the MMA kernel.
int gb_gemv_dot_rows(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                     int64_t workspace_bytes, void* stream);
int64_t gb_gemv_dot_rows_workspace_bytes(int64_t M, int64_t N, int64_t K);
int gb_gemv_dot(const void* x, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                int64_t workspace_bytes, void* stream);
int64_t gb_gemv_dot_workspace_bytes(int64_t N, int64_t K);

// ---------------------------------------------------------------------------
// scalar formats
// ---------------------------------------------------------------------------
GB_DEVINL float gb_bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

GB_DEVINL uint32_t gb_f32_to_bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Two fp32 -> one word of two bf16 (a in the low half), round to nearest even: one conversion.
GB_DEVINL uint32_t gb_pack_bf16x2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// E4M3 byte -> fp32, exact (no NaN handling: 0x7F/0xFF decode as 480, never stored).
GB_DEVINL float gb_e4m3_to_f32(uint32_t b) {
  const uint32_t mag = b & 0x7Fu;
  // place exponent+mantissa at the fp32 exponent, then rebias by 2^120; the
  // multiply also renormalises the subnormal codes (exponent field 0).
  float f = __uint_as_float(mag << 20) * 0x1p120f;
  return (b & 0x80u) ? -f : f;
}

// fp32 -> E4M3 with ONE rounding to nearest even (the hardware cvt may round
// twice through fp16).  |f| must be < 480; callers clamp to 448 first.
GB_DEVINL uint32_t gb_f32_to_e4m3(float f) {
  uint32_t u = __float_as_uint(f);
  const uint32_t sign = (u >> 24) & 0x80u;
  u &= 0x7FFFFFFFu;
  uint32_t r;
  if (u < (121u << 23)) {
    // below 2^-6 the result is subnormal with quantum 2^-9: adding 2^14 makes
    // the fp32 adder do the nearest-even rounding at exactly that quantum.
    const float shifted = __uint_as_float(u) + 16384.0f;
    r = __float_as_uint(shifted) - __float_as_uint(16384.0f);
  } else {
    const uint32_t odd = (u >> 20) & 1u;
    u += 0x7FFFFu + odd;            // round at bit 20
    r = (u >> 20) - (120u << 3);    // rebias exponent 127 -> 7
  }
  return (r & 0x7Fu) | sign;
}

// Round-to-nearest on the signed E2M1 grid {0, +-.5, +-1, +-1.5, +-2, +-3, +-4, +-6} with the
// reference's tie rule (gridbook/codec.py:248-260): the upper neighbour wins only when it is
// STRICTLY closer, so an exact midpoint goes to the lower (more negative) rung.
GB_DEVINL float gb_e2m1_rtn(float v) {
  constexpr float grid[15] = {-6.0f, -4.0f, -3.0f, -2.0f, -1.5f, -1.0f, -0.5f, 0.0f,
                              0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f};
  // hi = first rung >= v (bucketize, right = false; the top rung when there is none),
  // lo = the rung before it (the bottom rung when hi is the bottom).  Selects only: a
  // dynamically indexed table would live in local memory.
  float hi = grid[14], lo = grid[0];
#pragma unroll
  for (int i = 14; i >= 0; --i)
    if (grid[i] >= v) hi = grid[i];
#pragma unroll
  for (int i = 0; i < 15; ++i)
    if (!(grid[i] >= v)) lo = grid[i];
  return fabsf(__fsub_rn(hi, v)) < fabsf(__fsub_rn(v, lo)) ? hi : lo;
}

// Group-16 E2M1 bucket of sixteen bf16 values (eight packed words), in place.
GB_DEVINL void gb_fp4_group16_qdq(uint32_t (&w)[8], int scale_rule) {
  float v[16];
  float amax = 0.0f;
  bool has_nan = false;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = gb_bf16_bits_to_f32(w[i] & 0xFFFFu);
    v[2 * i + 1] = gb_bf16_bits_to_f32(w[i] >> 16);
    amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    has_nan |= isnan(v[2 * i]) || isnan(v[2 * i + 1]);
  }
  amax = fmaxf(amax, 1e-8f);
  float scale = scale_rule == GB_SCALE_RULE_DIV ? __fdiv_rn(amax, 6.0f) : __fmul_rn(amax, 1.0f / 6.0f);
  if (has_nan) scale = __int_as_float(0x7FC00000);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float q0 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v[2 * i], scale)), scale);
    const float q1 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v[2 * i + 1], scale)), scale);
    w[i] = gb_f32_to_bf16_bits(q0) | (gb_f32_to_bf16_bits(q1) << 16);
  }
}

// The same bucket with the group spread over eight consecutive lanes (lane % 8 = word of the
// group): every lane of the warp must call it.  Bit-identical to gb_fp4_group16_qdq: the
// maximum ignores NaNs and does not depend on the order, everything else is per value.
GB_DEVINL uint32_t gb_fp4_group16_qdq_lanes(uint32_t w, int scale_rule) {
  const float v0 = gb_bf16_bits_to_f32(w & 0xFFFFu), v1 = gb_bf16_bits_to_f32(w >> 16);
  float amax = fmaxf(fabsf(v0), fabsf(v1));
  uint32_t nan = (isnan(v0) || isnan(v1)) ? 1u : 0u;
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    nan |= __shfl_xor_sync(0xffffffffu, nan, o);
  }
  amax = fmaxf(amax, 1e-8f);
  float scale = scale_rule == GB_SCALE_RULE_DIV ? __fdiv_rn(amax, 6.0f) : __fmul_rn(amax, 1.0f / 6.0f);
  if (nan) scale = __int_as_float(0x7FC00000);
  const float q0 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v0, scale)), scale);
  const float q1 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v1, scale)), scale);
  return gb_f32_to_bf16_bits(q0) | (gb_f32_to_bf16_bits(q1) << 16);
}

// The same bucket with a group split over two adjacent lanes (eight values each, lane ^ 1 holds
// the other half): both lanes must call it.  Bit-identical to gb_fp4_group16_qdq.
GB_DEVINL uint4 gb_fp4_group16_qdq_pair(uint4 in, int scale_rule) {
  uint32_t w[4] = {in.x, in.y, in.z, in.w};
  float v[8];
  float amax = 0.0f;
  uint32_t nan = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = gb_bf16_bits_to_f32(w[i] & 0xFFFFu);
    v[2 * i + 1] = gb_bf16_bits_to_f32(w[i] >> 16);
    amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    nan |= (isnan(v[2 * i]) || isnan(v[2 * i + 1])) ? 1u : 0u;
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  nan |= __shfl_xor_sync(0xffffffffu, nan, 1);
  amax = fmaxf(amax, 1e-8f);
  float scale = scale_rule == GB_SCALE_RULE_DIV ? __fdiv_rn(amax, 6.0f) : __fmul_rn(amax, 1.0f / 6.0f);
  if (nan) scale = __int_as_float(0x7FC00000);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float q0 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v[2 * i], scale)), scale);
    const float q1 = __fmul_rn(gb_e2m1_rtn(__fdiv_rn(v[2 * i + 1], scale)), scale);
    w[i] = gb_f32_to_bf16_bits(q0) | (gb_f32_to_bf16_bits(q1) << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------
// bit-stream extraction (docs/SPEC.md:56-92): codeword c of a superblock
// occupies stream bits [c*k, c*k+k), least significant bit first.
// ---------------------------------------------------------------------------
// p must point at a 4-byte aligned address at or before the first needed byte;
// bit is the offset of the codeword's LSB from p (may exceed 31).
template <typename Ptr>
GB_DEVINL uint64_t gb_extract_bits(Ptr words, uint32_t bit, int k_bits) {
  const uint32_t w = bit >> 5, s = bit & 31u;
  const uint32_t a = words[w], b = words[w + 1];
  uint64_t lo = __funnelshift_r(a, b, s);
  if (k_bits > 32) {
    const uint32_t c = words[w + 2];
    lo |= (uint64_t)__funnelshift_r(b, c, s) << 32;
  }
  return k_bits >= 64 ? lo : (lo & ((1ull << k_bits) - 1ull));
}

// Generic byte-granular version for unaligned global rows (expand kernels).
GB_DEVINL uint64_t gb_extract_bits_bytes(const uint8_t* p, int64_t nbytes_valid,
                                         uint32_t bit, int k_bits) {
  const uint32_t byte0 = bit >> 3, s = bit & 7u;
  const int nb = (int)(s + (uint32_t)k_bits + 7u) >> 3;     // bytes the field touches
  uint64_t win = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t idx = (int64_t)byte0 + i;
    const uint64_t v = (i < nb && idx < nbytes_valid) ? (uint64_t)p[idx] : 0ull;
    win |= v << (8 * i);
  }
  return (win >> s) & ((1ull << k_bits) - 1ull);
}

struct GbSplit {
  int width[4];
  int shift[4];
  int base[4];   // element offset of sub-table i inside one codebook block
  int sub_dim;
  int n_sub;
};

__host__ __device__ inline GbSplit gb_make_split(int k_bits, int n_sub) {
  GbSplit s;
  s.n_sub = n_sub;
  s.sub_dim = 8 / n_sub;
  int off = 0, base = 0;
  for (int i = 0; i < 4; ++i) {
    if (i < n_sub) {
      s.width[i] = k_bits / n_sub + (i < k_bits % n_sub ? 1 : 0);
      s.shift[i] = off;
      s.base[i] = base;
      off += s.width[i];
      base += (1 << s.width[i]) * s.sub_dim;
    } else {
      s.width[i] = 0; s.shift[i] = 0; s.base[i] = 0;
    }
  }
  return s;
}

__host__ __device__ inline int64_t gb_codebook_elems(const gb_format& f) {
  if (f.mode == GB_MODE_FULL) return (int64_t)8 << f.k_bits;
  if (f.mode == GB_MODE_SIGNED) return (int64_t)8 << (f.k_bits - 8);
  GbSplit s = gb_make_split(f.k_bits, f.n_sub);
  return (int64_t)s.base[f.n_sub - 1] + ((int64_t)s.sub_dim << s.width[f.n_sub - 1]);
}

// ---------------------------------------------------------------------------
// mbarrier / bulk-copy primitives (all waits are bounded)
// ---------------------------------------------------------------------------
GB_DEVINL uint32_t gb_smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

GB_DEVINL void gb_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gb_smem_u32(bar)), "r"(count));
}

GB_DEVINL void gb_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gb_smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

GB_DEVINL void gb_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gb_smem_u32(bar)) : "memory");
}

// Programmatic dependent launch.  A kernel launched through gb_launch may start while the
// kernel before it on the stream is still running; gb_pdl_wait() returns once that kernel
// (and everything before it) has completed and its writes are visible, so it must come before
// the first read of anything an earlier kernel produced and before the first global write.
// What sits in front of it - barrier setup, the prefetch of weights, tables of constants -
// overlaps the predecessor's tail.  gb_pdl_launch_dependents() lets the successor start.
GB_DEVINL void gb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
GB_DEVINL void gb_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

GB_DEVINL uint64_t gb_globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Returns false when the wait ran out of patience (two seconds of wall clock);
// the caller raises the status word and leaves the kernel.
// `tok` (optional) receives a value the compiler cannot see through; loads that must not move
// above the wait take it as an operand.
GB_DEVINL bool gb_mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* tok = nullptr) {
  const uint32_t addr = gb_smem_u32(bar);
  uint64_t t0 = 0;
  if (tok) *tok = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) {
      if (tok) *tok = done;
      return true;
    }
    if ((spin & 255u) == 255u) {
      const uint64_t now = gb_globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
}

// 1-D bulk copy global -> this CTA's shared memory, completion on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
GB_DEVINL void gb_bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          gb_smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(gb_smem_u32(bar))
      : "memory");
}

GB_DEVINL void gb_fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// D[16x8] = A[16x8] . B[8x8] (bf16 in, fp32 out, no accumulator input)
GB_DEVINL void gb_mma_bf16_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

GB_DEVINL void gb_mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  // not volatile: a pure function of its register operands, free to be interleaved
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
