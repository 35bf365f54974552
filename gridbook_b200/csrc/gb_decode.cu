// Activation buckets and decoded-tile expanders.
//
// The expanders are the bit-exact gate of the whole library: every other kernel's
// decode reduces to "the tile it multiplies equals what these write".
#include "gb_common.cuh"

namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------
// Activation buckets (gridbook/codec.py:248-260, 428-437)
// ---------------------------------------------------------------------------
// One thread per group of 16: two 16-byte loads, amax, scale, 16 roundings.
__global__ void __launch_bounds__(kThreads)
fp4_group16_qdq_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out,
                       int64_t n_groups, int scale_rule) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + g * 16);
  const uint4 r0 = src[0], r1 = src[1];
  uint32_t packed[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
  gb_fp4_group16_qdq(packed, scale_rule);
  uint4* dst = reinterpret_cast<uint4*>(out + g * 16);
  dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// One block per token row: block-wide amax, then every element is scaled,
// rounded once to E4M3 and scaled back.
__global__ void __launch_bounds__(kThreads)
fp8_token_qdq_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int64_t K,
                     int scale_rule) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const uint16_t* row = x + (int64_t)blockIdx.x * K;
  uint16_t* orow = out + (int64_t)blockIdx.x * K;
  __shared__ float red[kThreads / 32];
  __shared__ float s_scale;
  float amax = 0.0f;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x)
    amax = fmaxf(amax, fabsf(gb_bf16_bits_to_f32(row[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int w = 1; w < kThreads / 32; ++w) a = fmaxf(a, red[w]);
    const float s = scale_rule == GB_SCALE_RULE_DIV ? __fdiv_rn(a, 448.0f)
                                                    : __fmul_rn(a, 1.0f / 448.0f);
    s_scale = fmaxf(s, 1.0f / (448.0f * 512.0f));
  }
  __syncthreads();
  const float scale = s_scale;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
    const float v = gb_bf16_bits_to_f32(row[i]);
    const float q = fminf(fmaxf(__fdiv_rn(v, scale), -448.0f), 448.0f);
    const float dq = gb_e4m3_to_f32(gb_f32_to_e4m3(q));
    orow[i] = (uint16_t)gb_f32_to_bf16_bits(__fmul_rn(dq, scale));
  }
}

// ---------------------------------------------------------------------------
// Expanders.  One warp per (row, superblock); lane v owns codeword v, i.e. the
// eight weights [8v, 8v+8) of the superblock and half of group v/2.
// ---------------------------------------------------------------------------
struct ExpandArgs {
  const uint8_t* qw;
  int64_t row_stride;
  int64_t valid_bytes;   // bytes that may be read from the first row's start
  const void* codebook;
  const int32_t* cb_row_offset;
  const float* compose;
  const float* weight_scale;   // fp8 grid: per-row scale, indexed by the absolute row
  int64_t row0, nrows, K;
  gb_format fmt;
  GbSplit split;
};

// Codebook values of one codeword as fp32 (exact for both grids).
template <bool kFp8>
GB_DEVINL void gather_values(const ExpandArgs& a, int64_t cb_base, uint64_t code, float (&val)[8]) {
  auto load = [&](int64_t idx) -> float {
    if constexpr (kFp8)
      return gb_e4m3_to_f32(reinterpret_cast<const uint8_t*>(a.codebook)[cb_base + idx]);
    else
      return gb_bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(a.codebook)[cb_base + idx]);
  };
  if (a.fmt.mode == GB_MODE_FULL) {
    if constexpr (!kFp8) {
      // a full codeword is eight consecutive bf16: one 16-byte load when the block is aligned
      const uint16_t* entry = reinterpret_cast<const uint16_t*>(a.codebook) + cb_base + (int64_t)code * 8;
      if ((reinterpret_cast<uintptr_t>(entry) & 15u) == 0) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(entry));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          val[2 * j] = gb_bf16_bits_to_f32(w[j] & 0xffffu);
          val[2 * j + 1] = gb_bf16_bits_to_f32(w[j] >> 16);
        }
        return;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) val[j] = load((int64_t)code * 8 + j);
  } else if (a.fmt.mode == GB_MODE_SIGNED) {
    const int64_t mag = (int64_t)(code >> 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float m = load(mag * 8 + j);
      val[j] = ((code >> j) & 1ull) ? -m : m;
    }
  } else {
    const int sd = a.split.sub_dim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = j / sd;   // sd is 2 or 4, so s < n_sub
      const int64_t idx = (int64_t)((code >> a.split.shift[s]) & ((1ull << a.split.width[s]) - 1ull));
      val[j] = load(a.split.base[s] + idx * sd + (j - s * sd));
    }
  }
}

// Group scale of codeword v (group v/2) for the fp4 grid, as fp32 and as its E4M3 byte.
GB_DEVINL float fp4_group_scale(const ExpandArgs& a, const uint8_t* sb, int v, uint32_t* byte_out) {
  const int g = v >> 1;
  const uint8_t* plane = sb + 4 * a.fmt.k_bits;
  if (a.fmt.scale_coding == GB_SCALE_V1) {
    const uint32_t b = plane[g];
    *byte_out = b;
    return gb_e4m3_to_f32(b);
  }
  const uint32_t e = plane[0];
  const uint32_t nib = (plane[1 + (g >> 1)] >> ((g & 1) * 4)) & 0xFu;
  const float s = a.compose[e * 16 + nib];
  *byte_out = gb_f32_to_e4m3(fminf(s, 448.0f));   // exact for every legal (E, c) pair
  return s;
}

enum { kOutFp8 = 0, kOutBf16 = 1, kOutNvfp4 = 2, kOutFp8Bf16 = 3 };

// Every warp takes kUnitsPerWarp consecutive (row, superblock) units and runs them in phases:
// all code loads, then all codebook and scale loads, then all stores, so that two independent
// load chains are in flight per lane.  Measured on the 805 MB bf16 tile of a 128-expert stack:
// one unit 327 us, two 291 us, four 372 us (fewer resident warps); at two the kernel writes
// 2.8 TB/s, close to the write half of a device copy.
constexpr int kUnitsPerWarp = 2;

template <int kOut>
__global__ void __launch_bounds__(kThreads)
expand_kernel(ExpandArgs a, void* __restrict__ out0, uint8_t* __restrict__ out_sf, int sf_swizzled) {
  constexpr bool kFp8Grid = kOut == kOutFp8 || kOut == kOutFp8Bf16;
  const int lane = threadIdx.x & 31;
  const int64_t n_sb = a.K / 256, units = a.nrows * n_sb;
  const int64_t unit0 = ((int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * kUnitsPerWarp;
  if (unit0 >= units) return;

  int64_t r[kUnitsPerWarp], s[kUnitsPerWarp];
  const uint8_t* sb[kUnitsPerWarp];
  uint64_t code[kUnitsPerWarp];
#pragma unroll
  for (int u = 0; u < kUnitsPerWarp; ++u) {
    const int64_t unit = unit0 + u < units ? unit0 + u : unit0;     // a dead unit re-reads the first
    // the unit index fits 32 bits whenever the grid does: one short division
    r[u] = unit < (1ll << 32) ? (int64_t)((uint32_t)unit / (uint32_t)n_sb) : unit / n_sb;
    s[u] = unit - r[u] * n_sb;
    const int64_t sb_off = r[u] * a.row_stride + s[u] * a.fmt.type_size;
    sb[u] = a.qw + sb_off;   // a.qw is the first byte of row0
    // byte-wide codes sit at byte `lane` of the superblock; other widths go through the bit window
    code[u] = a.fmt.k_bits == 8 ? (uint64_t)sb[u][lane]
                                : gb_extract_bits_bytes(sb[u], a.valid_bytes - sb_off, (uint32_t)(lane * a.fmt.k_bits),
                                                        a.fmt.k_bits);
  }

  float val[kUnitsPerWarp][8], scale[kUnitsPerWarp];
  uint32_t sbyte[kUnitsPerWarp];
  uint4 raw[kUnitsPerWarp];          // bf16 tile of a full-mode codeword: the eight bf16 as loaded
  bool have_raw[kUnitsPerWarp];
#pragma unroll
  for (int u = 0; u < kUnitsPerWarp; ++u) {
    const int64_t row = a.row0 + r[u];
    const int64_t cb_base = a.cb_row_offset ? (int64_t)a.cb_row_offset[row] : 0;
    have_raw[u] = false;
    if constexpr (kOut == kOutBf16) {
      const uint16_t* entry = reinterpret_cast<const uint16_t*>(a.codebook) + cb_base + (int64_t)code[u] * 8;
      if (a.fmt.mode == GB_MODE_FULL && (reinterpret_cast<uintptr_t>(entry) & 15u) == 0) {
        raw[u] = __ldg(reinterpret_cast<const uint4*>(entry));
        have_raw[u] = true;
      }
    }
    if (!have_raw[u]) gather_values<kFp8Grid>(a, cb_base, code[u], val[u]);
    sbyte[u] = 0;
    if constexpr (kOut == kOutFp8Bf16) scale[u] = a.weight_scale[row];     // the served weight's row scale
    else if constexpr (kOut == kOutFp8) scale[u] = 1.0f;
    else scale[u] = fp4_group_scale(a, sb[u], lane, &sbyte[u]);
  }

#pragma unroll
  for (int u = 0; u < kUnitsPerWarp; ++u) {
    if (unit0 + u >= units) break;
    const int64_t col = s[u] * 256 + lane * 8;
    const int64_t at = r[u] * a.K + col;
    if constexpr (kOut == kOutFp8) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= gb_f32_to_e4m3(val[u][j]) << (8 * j);
        hi |= gb_f32_to_e4m3(val[u][4 + j]) << (8 * j);
      }
      *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(out0) + at) = make_uint2(lo, hi);
    } else if constexpr (kOut == kOutBf16 || kOut == kOutFp8Bf16) {
      // bf16(value * scale): the group scale (fp4 grid) or the row scale (fp8 grid)
      uint32_t p[4];
      const uint32_t sbits = __float_as_uint(scale[u]);
      if (kOut == kOutBf16 && have_raw[u] && (sbits & 0xFFFFu) == 0) {
        // the scale is a bf16 number (every E4M3 byte is): the packed bf16 multiply rounds the
        // exact product once, the same bits as bf16(f32(value) * f32(scale))
        const uint32_t s2 = (sbits >> 16) * 0x10001u;
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p[j]) : "r"(w[j]), "r"(s2));
      } else {
        if (kOut == kOutBf16 && have_raw[u]) {
          const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            val[u][2 * j] = gb_bf16_bits_to_f32(w[j] & 0xffffu);
            val[u][2 * j + 1] = gb_bf16_bits_to_f32(w[j] >> 16);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          p[j] = gb_pack_bf16x2(__fmul_rn(val[u][2 * j], scale[u]), __fmul_rn(val[u][2 * j + 1], scale[u]));
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out0) + at) = make_uint4(p[0], p[1], p[2], p[3]);
    } else {
      uint32_t nib = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // E2M1 code: magnitudes {0,.5,1,1.5,2,3,4,6} -> 0..7, bit 3 = sign
        const float m = fabsf(val[u][j]);
        const uint32_t c = m < 2.0f ? (uint32_t)(m * 2.0f) : (m < 4.0f ? (uint32_t)m + 2u : (m < 6.0f ? 6u : 7u));
        nib |= (c | (val[u][j] < 0.0f ? 8u : 0u)) << (4 * j);
      }
      if (sf_swizzled == 2 && (sbyte[u] & 0x80u)) {
        // operand form of the block-scaled MMA, whose scale factors carry no sign: a negative
        // group scale moves its sign into the group's sixteen values, (-s) * v = s * (-v)
        nib ^= 0x88888888u;
        sbyte[u] &= 0x7Fu;
      }
      reinterpret_cast<uint32_t*>(out0)[at >> 3] = nib;
      if ((lane & 1) == 0) {
        const int64_t groups = a.K / 16;
        const int64_t g = s[u] * 16 + (lane >> 1);
        int64_t off = r[u] * groups + g;
        if (sf_swizzled) {
          const int64_t gpad = (groups + 3) / 4 * 4;
          const int64_t rr = r[u];
          off = (rr % 32) * 16 + ((rr / 32) % 4) * 4 + (g % 4) + (g / 4) * 512 + (rr / 128) * (512 * (gpad / 4));
        }
        out_sf[off] = (uint8_t)sbyte[u];
      }
    }
  }
}

int make_expand_args(const gb_weight* w, int64_t row0, int64_t nrows, ExpandArgs* a) {
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(row0 >= 0 && nrows > 0 && row0 + nrows <= w->rows, "rows [%lld, %lld) outside [0, %lld)",
             (long long)row0, (long long)(row0 + nrows), (long long)w->rows);
  a->qw = w->qw;
  a->row_stride = w->row_stride;
  a->codebook = w->codebook;
  a->cb_row_offset = w->cb_row_offset;
  a->compose = w->compose;
  a->weight_scale = w->weight_scale;
  a->row0 = row0;
  a->nrows = nrows;
  a->K = w->K;
  a->fmt = w->fmt;
  a->split = gb_make_split(w->fmt.k_bits, w->fmt.mode == GB_MODE_PRODUCT ? w->fmt.n_sub : 1);
  return GB_OK;
}

}  // namespace

extern "C" {

int gb_fp4_act_qdq(const void* x, void* out, int64_t M, int64_t K, int scale_rule, void* stream) {
  GB_REQUIRE(x && out, "null activation pointer");
  GB_REQUIRE(M >= 0 && K > 0 && K % 16 == 0, "fp4 activation bucket wants K %% 16 == 0, got K=%lld",
             (long long)K);
  if (M == 0) return GB_OK;
  const int64_t groups = M * (K / 16);
  const unsigned blocks = (unsigned)((groups + kThreads - 1) / kThreads);
  GB_CUDA_OK(gb_launch(fp4_group16_qdq_kernel, dim3(blocks), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const uint16_t*)x, (uint16_t*)out, groups, scale_rule));
  return GB_OK;
}

int gb_fp8_act_qdq(const void* x, void* out, int64_t M, int64_t K, int scale_rule, void* stream) {
  GB_REQUIRE(x && out, "null activation pointer");
  GB_REQUIRE(M >= 0 && K > 0, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (M == 0) return GB_OK;
  GB_CUDA_OK(gb_launch(fp8_token_qdq_kernel, dim3((unsigned)M), dim3(kThreads), 0, (cudaStream_t)stream,
                       (const uint16_t*)x, (uint16_t*)out, K, scale_rule));
  return GB_OK;
}

}  // extern "C"

namespace {
template <int kOut>
int launch_expand(const gb_weight* w, int64_t row0, int64_t nrows, void* out0, void* out_sf,
                  int sf_swizzled, void* stream) {
  ExpandArgs a;
  int rc = make_expand_args(w, row0, nrows, &a);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(out0 != nullptr, "null output");
  // The kernel addresses rows relative to row0 so that `valid_bytes` bounds every read.
  a.qw = w->qw + row0 * w->row_stride;
  a.valid_bytes = (nrows - 1) * w->row_stride + (w->K / 256) * w->fmt.type_size;
  const int64_t units = nrows * (w->K / 256);
  const int64_t per_cta = (kThreads / 32) * kUnitsPerWarp;
  const unsigned blocks = (unsigned)((units + per_cta - 1) / per_cta);
  gb_count_launch();
  expand_kernel<kOut><<<blocks, kThreads, 0, (cudaStream_t)stream>>>(a, out0, (uint8_t*)out_sf,
                                                                    sf_swizzled);
  GB_LAUNCH_OK("expand_kernel");
  return GB_OK;
}

// ---- the literal format's native NVFP4 view, fast -------------------------------------------
// Full mode, k = 8, E4M3-direct scales, one codebook: a codeword is one byte and its eight E2M1
// values are one 32-bit word of a 256-entry table kept in shared memory.  Eight lanes take one
// (row, superblock): each loads four codes as one word, looks them up and stores sixteen bytes
// (128 contiguous bytes per unit); the first four of them also write the unit's sixteen group
// scales, one word per 128 x 4 atom.  Memory-bound: 48 bytes read and 144 written per 256 weights.
constexpr int kLitUnroll = 4;                              // steps in flight per warp, four units each

__global__ void __launch_bounds__(kThreads)
expand_literal_nvfp4_kernel(const uint8_t* __restrict__ qw, int64_t row_stride, const uint16_t* __restrict__ codebook,
                            int64_t nrows, int64_t n_sb, uint4* __restrict__ out_packed,
                            uint8_t* __restrict__ out_sf, int fold_sign) {
  __shared__ uint32_t lut[256];
  {
    const uint4 e = __ldg(reinterpret_cast<const uint4*>(codebook) + threadIdx.x);     // kThreads == 256 entries
    const uint32_t w[4] = {e.x, e.y, e.z, e.w};
    uint32_t nib = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = gb_bf16_bits_to_f32((w[j >> 1] >> (16 * (j & 1))) & 0xffffu);
      const float m = fabsf(v);
      const uint32_t c = m < 2.0f ? (uint32_t)(m * 2.0f) : (m < 4.0f ? (uint32_t)m + 2u : (m < 6.0f ? 6u : 7u));
      nib |= (c | (v < 0.0f ? 8u : 0u)) << (4 * j);
    }
    lut[threadIdx.x] = nib;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, sub = lane & 7, which = lane >> 3;
  const int64_t units = nrows * n_sb;
  const int64_t k_atoms = n_sb * 4;                        // atoms along K of one 128-row tile
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t u0 = ((int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * (4 * kLitUnroll); u0 < units;
       u0 += warps * (4 * kLitUnroll)) {
    uint32_t codes[kLitUnroll], sc2[kLitUnroll], sc4[kLitUnroll];
#pragma unroll
    for (int i = 0; i < kLitUnroll; ++i) {
      const int64_t u = u0 + 4 * i + which < units ? u0 + 4 * i + which : u0;
      const int64_t r = u / n_sb, sb = u - r * n_sb;
      const uint8_t* p = qw + r * row_stride + sb * 48;    // 16-byte aligned: rows are, and 48 is a multiple of 16
      codes[i] = __ldg(reinterpret_cast<const uint32_t*>(p) + sub);
      sc2[i] = __ldg(reinterpret_cast<const uint16_t*>(p + 32) + sub);                      // groups 2 sub, 2 sub + 1
      sc4[i] = sub < 4 ? __ldg(reinterpret_cast<const uint32_t*>(p + 32) + sub) : 0u;       // the scales of atom `sub`
    }
#pragma unroll
    for (int i = 0; i < kLitUnroll; ++i) {
      const int64_t u = u0 + 4 * i + which;
      if (u >= units) continue;
      const int64_t r = u / n_sb, sb = u - r * n_sb;
      uint32_t w0 = lut[codes[i] & 0xffu], w1 = lut[(codes[i] >> 8) & 0xffu];
      uint32_t w2 = lut[(codes[i] >> 16) & 0xffu], w3 = lut[codes[i] >> 24];
      if (fold_sign) {
        if (sc2[i] & 0x80u) { w0 ^= 0x88888888u; w1 ^= 0x88888888u; }
        if (sc2[i] & 0x8000u) { w2 ^= 0x88888888u; w3 ^= 0x88888888u; }
      }
      out_packed[u * 8 + sub] = make_uint4(w0, w1, w2, w3);
      if (sub < 4) {
        const int64_t off = (r / 128) * (512 * k_atoms) + (sb * 4 + sub) * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4;
        *reinterpret_cast<uint32_t*>(out_sf + off) = fold_sign ? (sc4[i] & 0x7F7F7F7Fu) : sc4[i];
      }
    }
  }
}

int launch_expand_literal(const gb_weight* w, int64_t row0, int64_t nrows, void* out_packed, void* out_sf,
                          int fold_sign, void* stream) {
  const int64_t n_sb = w->K / 256, units = nrows * n_sb;
  const int64_t per_cta = (kThreads / 32) * 4 * kLitUnroll;
  int64_t blocks = (units + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)gb_sm_count() * 16;
  if (cap > 0 && blocks > cap) blocks = cap;
  gb_count_launch();
  expand_literal_nvfp4_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
      w->qw + row0 * w->row_stride, w->row_stride, (const uint16_t*)w->codebook, nrows, n_sb, (uint4*)out_packed,
      (uint8_t*)out_sf, fold_sign);
  GB_LAUNCH_OK("expand_literal_nvfp4_kernel");
  return GB_OK;
}
// The fp8 product formats k = 32 (four sub-tables of two values) and k = 16 (two sub-tables of four
// values) -> the E4M3 value plane, one byte per weight: the sub-table entries are copied through as
// they are.  Eight lanes per (row, superblock); a lane takes two codewords of each half of the
// superblock, so that every store instruction of the eight lanes writes 128 contiguous bytes.  The
// sub-tables sit in shared memory as 32-bit words, eight copies each (copy = lane mod 8: lanes of
// different copies never share a bank).  Memory-bound: 128 or 64 bytes read and 256 written per
// 256 weights.
constexpr int kF8Unroll = 4;

template <bool kK32>
__global__ void __launch_bounds__(kThreads)
expand_fp8_fast_kernel(const uint8_t* __restrict__ qw, int64_t row_stride, const uint8_t* __restrict__ codebook,
                       int64_t nrows, int64_t n_sb, uint4* __restrict__ out) {
  constexpr int kEntries = kK32 ? 1024 : 512;              // 4 x 256 two-byte or 2 x 256 four-byte entries
  constexpr int kSb = kK32 ? 128 : 64;
  __shared__ uint32_t lut[kEntries * 8];
  for (int e = threadIdx.x; e < kEntries; e += kThreads) {
    const uint32_t v = kK32 ? (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(codebook) + e)
                            : __ldg(reinterpret_cast<const uint32_t*>(codebook) + e);
#pragma unroll
    for (int j = 0; j < 8; ++j) lut[e * 8 + j] = v;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, sub = lane & 7, which = lane >> 3;
  const uint32_t* my = lut + sub;
  const int64_t units = nrows * n_sb;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t u0 = ((int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * (4 * kF8Unroll); u0 < units;
       u0 += warps * (4 * kF8Unroll)) {
    uint32_t in[kF8Unroll][kK32 ? 4 : 2];                  // two codewords of the first half, two of the second
#pragma unroll
    for (int i = 0; i < kF8Unroll; ++i) {
      const int64_t u = u0 + 4 * i + which < units ? u0 + 4 * i + which : u0;
      const int64_t r = u / n_sb, sb = u - r * n_sb;
      const uint8_t* p = qw + r * row_stride + sb * kSb;
      if (kK32) {
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(p) + sub), b = __ldg(reinterpret_cast<const uint2*>(p + 64) + sub);
        in[i][0] = a.x; in[i][1] = a.y; in[i][2] = b.x; in[i][3] = b.y;
      } else {
        in[i][0] = __ldg(reinterpret_cast<const uint32_t*>(p) + sub);
        in[i][1] = __ldg(reinterpret_cast<const uint32_t*>(p + 32) + sub);
      }
    }
#pragma unroll
    for (int i = 0; i < kF8Unroll; ++i) {
      const int64_t u = u0 + 4 * i + which;
      if (u >= units) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 o;
        if (kK32) {
          const uint32_t c0 = in[i][2 * half], c1 = in[i][2 * half + 1];
          o.x = my[(c0 & 0xffu) * 8] | (my[(256 + ((c0 >> 8) & 0xffu)) * 8] << 16);
          o.y = my[(512 + ((c0 >> 16) & 0xffu)) * 8] | (my[(768 + (c0 >> 24)) * 8] << 16);
          o.z = my[(c1 & 0xffu) * 8] | (my[(256 + ((c1 >> 8) & 0xffu)) * 8] << 16);
          o.w = my[(512 + ((c1 >> 16) & 0xffu)) * 8] | (my[(768 + (c1 >> 24)) * 8] << 16);
        } else {
          const uint32_t c = in[i][half];                  // two 16-bit codewords
          o.x = my[(c & 0xffu) * 8];
          o.y = my[(256 + ((c >> 8) & 0xffu)) * 8];
          o.z = my[((c >> 16) & 0xffu) * 8];
          o.w = my[(256 + (c >> 24)) * 8];
        }
        out[u * 16 + half * 8 + sub] = o;
      }
    }
  }
}

int launch_expand_fp8_fast(const gb_weight* w, int64_t row0, int64_t nrows, void* out, void* stream) {
  const bool k32 = w->fmt.k_bits == 32;
  const int64_t n_sb = w->K / 256, units = nrows * n_sb;
  const int64_t per_cta = (kThreads / 32) * 4 * kF8Unroll;
  int64_t blocks = (units + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)gb_sm_count() * 8;
  if (cap > 0 && blocks > cap) blocks = cap;
  gb_count_launch();
  const uint8_t* base = w->qw + row0 * w->row_stride;
  if (k32)
    expand_fp8_fast_kernel<true><<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
        base, w->row_stride, (const uint8_t*)w->codebook, nrows, n_sb, (uint4*)out);
  else
    expand_fp8_fast_kernel<false><<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
        base, w->row_stride, (const uint8_t*)w->codebook, nrows, n_sb, (uint4*)out);
  GB_LAUNCH_OK("expand_fp8_fast_kernel");
  return GB_OK;
}
}  // namespace

extern "C" {

int gb_expand_fp8(const gb_weight* w, int64_t row0, int64_t nrows, void* out, void* stream) {
  GB_REQUIRE(w && w->fmt.grid == GB_GRID_FP8, "gb_expand_fp8 wants an fp8-grid weight");
  const gb_format& f = w->fmt;
  if (f.mode == GB_MODE_PRODUCT && ((f.k_bits == 32 && f.n_sub == 4 && f.type_size == 128) ||
                                    (f.k_bits == 16 && f.n_sub == 2 && f.type_size == 64)) &&
      w->cb_row_offset == nullptr && ((uintptr_t)w->codebook & 3u) == 0 && ((uintptr_t)out & 15u) == 0 &&
      ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0) {
    int rc = gb_check_weight(w);
    if (rc != GB_OK) return rc;
    GB_REQUIRE(out != nullptr, "null output pointer");
    GB_REQUIRE(row0 >= 0 && nrows >= 0 && row0 + nrows <= w->rows, "rows [%lld, %lld) outside [0, %lld)",
               (long long)row0, (long long)(row0 + nrows), (long long)w->rows);
    if (nrows == 0) return GB_OK;
    return launch_expand_fp8_fast(w, row0, nrows, out, stream);
  }
  return launch_expand<kOutFp8>(w, row0, nrows, out, nullptr, 0, stream);
}

int gb_expand_fp8_bf16(const gb_weight* w, int64_t row0, int64_t nrows, void* out, void* stream) {
  GB_REQUIRE(w && w->fmt.grid == GB_GRID_FP8 && w->weight_scale, "gb_expand_fp8_bf16 wants an fp8-grid weight with its row scales");
  return launch_expand<kOutFp8Bf16>(w, row0, nrows, out, nullptr, 0, stream);
}

int gb_expand_fp4_bf16(const gb_weight* w, int64_t row0, int64_t nrows, void* out, void* stream) {
  GB_REQUIRE(w && w->fmt.grid == GB_GRID_FP4, "gb_expand_fp4_bf16 wants an fp4-grid weight");
  return launch_expand<kOutBf16>(w, row0, nrows, out, nullptr, 0, stream);
}

int gb_expand_fp4_nvfp4(const gb_weight* w, int64_t row0, int64_t nrows, void* out_packed,
                        void* out_sf, int sf_swizzled, void* stream) {
  GB_REQUIRE(w && w->fmt.grid == GB_GRID_FP4, "gb_expand_fp4_nvfp4 wants an fp4-grid weight");
  GB_REQUIRE(out_sf != nullptr, "null scale-factor output");
  const gb_format& f = w->fmt;
  if (sf_swizzled != 0 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
      w->cb_row_offset == nullptr && ((uintptr_t)w->codebook & 15u) == 0 && ((uintptr_t)out_packed & 15u) == 0 &&
      ((uintptr_t)out_sf & 3u) == 0 && ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0 && kThreads == 256) {
    int rc = gb_check_weight(w);
    if (rc != GB_OK) return rc;
    GB_REQUIRE(out_packed != nullptr, "null output pointer");
    GB_REQUIRE(row0 >= 0 && nrows >= 0 && row0 + nrows <= w->rows, "rows [%lld, %lld) outside [0, %lld)",
               (long long)row0, (long long)(row0 + nrows), (long long)w->rows);
    if (nrows == 0) return GB_OK;
    return launch_expand_literal(w, row0, nrows, out_packed, out_sf, sf_swizzled == 2, stream);
  }
  return launch_expand<kOutNvfp4>(w, row0, nrows, out_packed, out_sf, sf_swizzled, stream);
}

}  // extern "C"
