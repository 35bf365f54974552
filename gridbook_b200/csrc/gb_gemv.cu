// Decode-batch (M <= 16) codebook linear and grouped routed-MoE GEMV.
//
// Persistent CTAs of eight warps walk tiles of 64 output rows (x one K slice).  Every
// warp owns eight whole rows of the tile and streams them through a private
// shared-memory ring with 1-D bulk copies (16-byte aligned windows around rows of any
// stride, so odd type_size rows need no repacking; each row lands on a bank-skewed
// pitch).  The ring is refilled by the warp itself as soon as a stage is consumed, so
// in steady state there is no CTA-wide synchronisation at all.  Lane (g, t) expands
// codewords t, 4+t, ... of every superblock of row g through a shared-memory codebook
// into bf16 grid values times the group scale (exact: <= 6 significant bits) and feeds
// them to m16n8k16 bf16 MMAs against the activation rows held in shared memory; the
// accumulators are scaled and rounded to bf16 once.  K slices (only when the activation
// rows or a warp's rows would not fit) add into an fp32 workspace instead.
#include "gb_common.cuh"

#include <atomic>
#include <mutex>

namespace {

constexpr int kMaxWarps = 16;             // the literal fast path (128 registers) runs 16 warps, the rest 8
constexpr int kMaxStages = 4;
constexpr int kSmemBig = 216 * 1024;      // one CTA per SM
constexpr int kXBudget = 64 * 1024;
constexpr uint32_t kExpBias120 = 120u << 7;   // bf16 exponent offset of 2^120

enum Fmt { kFp4Prod2 = 0, kFp4Signed = 1, kFp4Full = 2, kFp8Prod4 = 3, kFp8Prod2 = 4, kNumFmt = 5 };

struct GemvParams {
  // activations
  const uint16_t* x;      // [rows, K] bf16
  const int32_t* x_row;   // MoE: activation row of pair p (NULL = p)
  int M;                  // dense: number of activation rows
  // weights
  const uint8_t* qw;
  int64_t row_stride;
  int64_t expert_stride;  // bytes between experts (MoE)
  const void* codebook;
  const int32_t* cb_row_offset;
  const float* compose;
  const float* weight_scale;
  float global_scale;
  int64_t N, K;
  gb_format fmt;
  GbSplit split;
  int cb_elems;           // scalars in one codebook block
  // routing (MoE)
  const int32_t* offsets;
  const int32_t* order;
  int E;
  int swiglu;             // tile = 4 gate rows + 4 up rows, output silu(g)*u
  int act, scale_rule;    // routed: fp4 group-16 bucket applied while the activation rows are staged
  int m_chunk;            // tokens per tile pass (MoE), <= 16
  // tiling
  int ksplit, sb_per_slice, n_sb;
  int sb_per_chunk;       // a warp streams its rows through the ring in chunks of this many superblocks
  int warps;              // warps per CTA (8 or 16); a tile is 8 * warps rows
  int n_row_tiles;
  int stages, stage_bytes, row_pitch;
  int x_pitch;            // bytes between activation rows in shared memory
  int x_rows;             // activation rows staged (1..16); MMA rows beyond them are zero
  int lut_bytes;
  int etab_bytes;         // routed: shared-memory bytes of the per-expert tile prefix and offsets
  int lut_rep;            // copies of each 16-byte table entry (1 or 8): lane l reads copy l % 8, so the
                          // eight lanes of a quarter-warp never collide on a bank
  // outputs
  uint16_t* y;
  uint16_t* y_peer[8];    // routed, optional: pair p's row lives in y_peer[p / pairs_per_rank]
  int pairs_per_rank;     // 0 = all rows in y
  float* ws;              // [M, N] fp32 partial sums when ksplit > 1
  int* status;
};

struct Tile {
  int row0;       // first output row (gate row for swiglu)
  int nrows;      // valid rows in the (half) tile
  int expert;
  int m0, mcount; // sorted-pair range of this pass (MoE) or [0, M)
  int slice;
  int chunk, nchunks;   // this step's K chunk of the slice; accumulators live across a tile's chunks
};

// Every thread of the CTA enumerates the same tile sequence.
template <bool kMoE>
struct TileWalker {
  const GemvParams& p;
  int next_local;   // dense: next row-tile index; MoE: next global tile index for this CTA
  int e, base;      // MoE: current expert and the global index of its first tile
  int last = 0;     // MoE: one past this CTA's last tile
  const int* tile_base;   // MoE, shared memory: [E + 1] first global tile index of every expert
  const int* offs;        // MoE, shared memory: [E + 1] copy of the routing offsets
  __device__ TileWalker(const GemvParams& pp, const int* tb, const int* of) : p(pp), tile_base(tb), offs(of) {
    if constexpr (kMoE) {
      // A CTA takes a contiguous run of the global tile list: consecutive tiles are mostly row
      // tiles of the same (expert, token pass), whose activation rows are then staged once.
      const int total = tile_base[p.E];
      const int run = (total + (int)gridDim.x - 1) / (int)gridDim.x;
      next_local = (int)blockIdx.x * run;
      last = min(total, next_local + run);
      e = 0; base = 0;
    } else {
      next_local = blockIdx.x / p.ksplit;
    }
  }
  __device__ bool next_tile(Tile& t) {
    const int tile_rows = 8 * p.warps;
    if constexpr (!kMoE) {
      if (next_local >= p.n_row_tiles) return false;
      t.row0 = next_local * tile_rows;
      t.nrows = min(tile_rows, (int)(p.N - t.row0));
      t.expert = 0; t.m0 = 0; t.mcount = p.M;
      t.slice = blockIdx.x % p.ksplit;
      next_local += gridDim.x / p.ksplit;
      return true;
    } else {
      const int half = p.swiglu ? tile_rows / 2 : tile_rows;
      if (next_local >= last) return false;
      // the expert whose tile range holds next_local: the last e with tile_base[e] <= next_local
      // (experts without tokens have empty ranges and are skipped by the search)
      int lo = e, hi = p.E;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_base[mid] <= next_local) lo = mid; else hi = mid;
      }
      e = lo;
      {
        const int cnt = offs[e + 1] - offs[e];
        const int local = next_local - tile_base[e];
        const int ch = local / p.n_row_tiles, rt = local - ch * p.n_row_tiles;
        const int rows_out = p.swiglu ? (int)(p.N / 2) : (int)p.N;
        t.row0 = rt * half;
        t.nrows = min(half, rows_out - t.row0);
        t.expert = e;
        t.m0 = offs[e] + ch * p.m_chunk;
        t.mcount = min(p.m_chunk, cnt - ch * p.m_chunk);
        t.slice = 0;
        next_local += 1;
        return true;
      }
      return false;
    }
  }
  // One step = one K chunk of one tile; a tile's chunks come back to back.
  Tile cur;
  bool have = false;
  __device__ bool next(Tile& t) {
    if (have && cur.chunk + 1 < cur.nchunks) {
      ++cur.chunk;
    } else {
      if (!next_tile(cur)) return false;
      const int nsb = min(p.sb_per_slice, p.n_sb - cur.slice * p.sb_per_slice);
      cur.chunk = 0;
      cur.nchunks = (nsb + p.sb_per_chunk - 1) / p.sb_per_chunk;
      have = true;
    }
    t = cur;
    return true;
  }
};

// Row g (0..7) of warp `warp`'s share of a tile: its first byte in global memory, or
// nullptr past the edge.  With swiglu a warp takes four gate rows and the four matching
// up rows, so a tile covers 32 gate rows + 32 up rows.
GB_DEVINL const uint8_t* tile_row_ptr(const GemvParams& p, const Tile& t, int warp, int g, int64_t* out_row) {
  int local = 8 * warp + g;
  int64_t row = (int64_t)t.row0 + local;
  if (p.swiglu) {
    local = 4 * warp + (g & 3);
    row = (int64_t)t.row0 + local + (g >= 4 ? p.N / 2 : 0);
  }
  *out_row = row;
  if (local >= t.nrows) return nullptr;
  return p.qw + (int64_t)t.expert * p.expert_stride + row * p.row_stride +
         ((int64_t)t.slice * p.sb_per_slice + (int64_t)t.chunk * p.sb_per_chunk) * p.fmt.type_size;
}

// shared-memory loads by 32-bit shared address
GB_DEVINL uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
GB_DEVINL uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
GB_DEVINL uint32_t lds_u16(uint32_t a) {
  uint32_t v;
  asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
  return v;
}
GB_DEVINL uint2 lds_v2(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
GB_DEVINL uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// Hot-loop loads.  They are NOT volatile, so the compiler may batch and interleave them; the
// extra `tok` operand is a value produced by the mbarrier wait of the current task, which
// keeps every such load after that wait (and after the activation restage before it) and
// makes loads of different tasks distinct expressions.
GB_DEVINL uint4 ldt_v4(uint32_t a, uint32_t tok) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4]; // %5" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "r"(tok));
  return v;
}
GB_DEVINL uint4 ldt_v4_if(uint32_t a, bool live, uint32_t tok) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  asm("{ .reg .pred q; setp.ne.u32 q, %5, 0; @q ld.shared.v4.u32 {%0,%1,%2,%3}, [%4]; } // %6"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "r"(a), "r"((uint32_t)live), "r"(tok));
  return v;
}

// 16-byte shared load that only lanes with `live` perform; the others get zeros and cost
// no shared-memory bandwidth.
GB_DEVINL uint4 lds_v4_if(uint32_t a, bool live) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  asm volatile(
      "{ .reg .pred q; setp.ne.u32 q, %5, 0; @q ld.shared.v4.u32 {%0,%1,%2,%3}, [%4]; }"
      : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
      : "r"(a), "r"((uint32_t)live));
  return v;
}

GB_DEVINL uint32_t mul_bf16x2(uint32_t a, uint32_t s2) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(s2));
  return d;
}

// Per-thread constants of the decode, computed once.
struct LaneDecode {
  uint32_t bit0;               // stream bit of this lane's first codeword (codeword t of the superblock)
  uint32_t kstep;              // stream bits between this lane's consecutive codewords (4 codewords)
  uint32_t mask[4], shift[4], lbase[4];   // product split: index masks, shifts, table byte offsets
  uint32_t scale_off;          // byte offset of the scale plane inside a superblock
  uint32_t ent_shift, rep_off; // 16-byte-entry tables: log2 of the entry pitch, this lane's replica offset
};

// Codeword bits at stream bit `bit` of the superblock at shared address sbp (any alignment).
template <bool kWide>
GB_DEVINL void fetch_code(uint32_t sbp, uint32_t bit, uint32_t& lo, uint32_t& hi) {
  const uint32_t a = sbp + (bit >> 3);
  const uint32_t mis = a & 3u, a4 = a - mis, sh = mis * 8u + (bit & 7u);
  const uint32_t w0 = lds_u32(a4), w1 = lds_u32(a4 + 4);
  lo = __funnelshift_r(w0, w1, sh);
  hi = 0;
  if constexpr (kWide) {
    const uint32_t w2 = lds_u32(a4 + 8);
    hi = __funnelshift_r(w1, w2, sh);
  }
}

// Expand one codeword through the shared-memory table into eight bf16 values.
template <int kFmt, bool kWide>
GB_DEVINL void expand_code(const LaneDecode& d, uint32_t lut, uint32_t lo, uint32_t hi, uint32_t (&w)[4]) {
  if constexpr (kFmt == kFp4Full) {
    const uint4 v = lds_v4(lut + ((lo & d.mask[0]) << d.ent_shift) + d.rep_off);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (kFmt == kFp4Signed) {
    const uint32_t code = lo & d.mask[0];
    const uint4 v = lds_v4(lut + ((code >> 8) << d.ent_shift) + d.rep_off);
    // sign bit j flips coordinate j: bit 15 of the low half, bit 31 of the high half
    w[0] = v.x ^ ((code & 1u) << 15) ^ ((code & 2u) << 30);
    w[1] = v.y ^ ((code & 4u) << 13) ^ ((code & 8u) << 28);
    w[2] = v.z ^ ((code & 16u) << 11) ^ ((code & 32u) << 26);
    w[3] = v.w ^ ((code & 64u) << 9) ^ ((code & 128u) << 24);
  } else if constexpr (kFmt == kFp4Prod2 || kFmt == kFp8Prod2) {
    const uint32_t i0 = lo & d.mask[0];
    const uint32_t i1 = (lo >> d.shift[1]) & d.mask[1];
    const uint2 va = lds_v2(lut + (i0 << 3));
    const uint2 vb = lds_v2(lut + d.lbase[1] + (i1 << 3));
    w[0] = va.x; w[1] = va.y; w[2] = vb.x; w[3] = vb.y;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t idx;
      if constexpr (kWide) {
        const uint64_t code = ((uint64_t)hi << 32) | lo;
        idx = (uint32_t)(code >> d.shift[i]) & d.mask[i];
      } else {
        idx = (lo >> d.shift[i]) & d.mask[i];
      }
      w[i] = lds_u32(lut + d.lbase[i] + (idx << 2));
    }
  }
}

// Same job when the rows of one task use different codebook blocks: gather this row's
// entries from global memory (rare: only tasks that straddle a role boundary).
template <bool kFp8>
GB_DEVINL void expand_code_global(const GemvParams& p, int64_t cb_off, uint32_t lo, uint32_t hi, uint32_t (&w)[4]) {
  uint64_t code = (uint64_t)lo | ((uint64_t)hi << 32);
  code &= (1ull << p.fmt.k_bits) - 1ull;
  const int sd = p.split.sub_dim;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t half[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = 2 * j + h;
      int64_t idx;
      bool neg = false;
      if (p.fmt.mode == GB_MODE_FULL) idx = (int64_t)code * 8 + c;
      else if (p.fmt.mode == GB_MODE_SIGNED) { idx = (int64_t)(code >> 8) * 8 + c; neg = (code >> c) & 1ull; }
      else {
        const int si = c / sd;
        idx = p.split.base[si] + (int64_t)((code >> p.split.shift[si]) & ((1ull << p.split.width[si]) - 1ull)) * sd + (c - si * sd);
      }
      uint32_t b;
      if constexpr (kFp8) b = __float_as_uint(gb_e4m3_to_f32(reinterpret_cast<const uint8_t*>(p.codebook)[cb_off + idx])) >> 16;
      else b = reinterpret_cast<const uint16_t*>(p.codebook)[cb_off + idx];
      if (neg) b ^= 0x8000u;
      if constexpr (!kFp8) {          // match the pre-scaled shared-memory table (values * 2^120)
        if (p.fmt.scale_coding == GB_SCALE_V1 && (b & 0x7FFFu)) b += kExpBias120;
      }
      half[h] = b;
    }
    w[j] = half[0] | (half[1] << 16);
  }
}

// A task whose eight rows use different codebook blocks (it straddles a role boundary of a
// fused module): same arithmetic, entries gathered from global memory.  Kept out of line so
// the common loop stays small.
template <bool kFp8>
__device__ __noinline__ void mixed_codebook_task(const GemvParams& p, const LaneDecode& d, uint32_t sbp, int nsb,
                                                 int64_t cb_off, float row_scale, uint32_t xa_s, uint32_t xb_s,
                                                 uint32_t xa_step, uint32_t xb_step, uint32_t sub_s, int t4,
                                                 float (&acc0)[4], float (&acc1)[4]) {
  const uint32_t ts = (uint32_t)p.fmt.type_size;
  const bool v1 = p.fmt.scale_coding == GB_SCALE_V1;
  for (int sb = 0; sb < nsb; ++sb, sbp += ts, xa_s += xa_step, xb_s += xb_step) {
    for (int kb = 0; kb < 8; ++kb) {
      const uint4 xa = lds_v4(xa_s + kb * 64);
      const uint4 xb = lds_v4(xb_s + kb * 64);
      uint32_t lo, hi, w[4];
      fetch_code<true>(sbp, d.bit0 + kb * d.kstep, lo, hi);
      expand_code_global<kFp8>(p, cb_off, lo, hi, w);
      if constexpr (kFp8) {
        for (int j = 0; j < 4; ++j) {
          const float flo = __uint_as_float(w[j] << 16) * row_scale;
          const float fhi = __uint_as_float(w[j] & 0xFFFF0000u) * row_scale;
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[j]) : "f"(fhi), "f"(flo));
        }
      } else {
        const uint32_t grp = 2u * kb + ((uint32_t)t4 >> 1);
        uint32_t sbits;
        if (v1) {
          const uint32_t b = lds_u8(sbp + d.scale_off + grp);
          sbits = ((b & 0x7Fu) << 4) | ((b & 0x80u) << 8);
        } else {
          const uint32_t e = lds_u8(sbp + d.scale_off);
          const uint32_t nib = (lds_u8(sbp + d.scale_off + 1u + (grp >> 1)) >> ((grp & 1u) * 4u)) & 0xFu;
          sbits = (lds_u16(sub_s + nib * 2u) + ((e - 127u) << 7)) & 0xFFFFu;
        }
        const uint32_t s2 = sbits * 0x10001u;
        for (int j = 0; j < 4; ++j) w[j] = mul_bf16x2(w[j], s2);
      }
      const uint32_t a0[4] = {xa.x, xb.x, xa.y, xb.y};
      const uint32_t a1[4] = {xa.z, xb.z, xa.w, xb.w};
      gb_mma_bf16_16816(acc0, a0, w[0], w[1]);
      gb_mma_bf16_16816(acc1, a1, w[2], w[3]);
    }
  }
}

// Copy one codebook block into the shared-memory table as bf16.  For the fp4 grid with
// E4M3-direct scales the entries are stored times 2^120, so that the raw scale byte,
// shifted into the bf16 exponent/mantissa field (= scale * 2^-120, subnormal codes
// included), multiplies to the exact product with one packed bf16 multiply.
template <int kFmt>
GB_DEVINL void stage_lut(const GemvParams& p, uint8_t* lut, int64_t cb_off, int tid, int nthreads) {
  constexpr bool fp8 = (kFmt == kFp8Prod4 || kFmt == kFp8Prod2);
  uint16_t* dst = reinterpret_cast<uint16_t*>(lut);
  if constexpr (fp8) {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.codebook) + cb_off;
    for (int i = tid; i < p.cb_elems; i += nthreads)
      dst[i] = (uint16_t)(__float_as_uint(gb_e4m3_to_f32(src[i])) >> 16);   // exact: 4 significant bits
  } else {
    const uint16_t* src = reinterpret_cast<const uint16_t*>(p.codebook) + cb_off;
    const uint32_t bias = p.fmt.scale_coding == GB_SCALE_V1 ? kExpBias120 : 0u;
    if (p.lut_rep > 1) {
      // entry e (eight values, 16 bytes) -> eight copies at (e * 8 + r) * 16 bytes
      const uint32_t bias2 = bias | (bias << 16);
      for (int i = tid; i < (p.cb_elems / 8) * 8; i += nthreads) {
        const int e = i >> 3, r = i & 7;
        uint4 v = *reinterpret_cast<const uint4*>(src + e * 8);
        uint32_t* q = &v.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t nz = ((q[j] & 0x7FFFu) ? 0xFFFFu : 0u) | ((q[j] & 0x7FFF0000u) ? 0xFFFF0000u : 0u);
          q[j] += bias2 & nz;
        }
        reinterpret_cast<uint4*>(lut)[e * 8 + r] = v;
      }
    } else {
      for (int i = tid; i < p.cb_elems; i += nthreads) {
        const uint32_t b = src[i];
        dst[i] = (uint16_t)((b & 0x7FFFu) ? b + bias : b);
      }
    }
  }
}

// Lanes 0..7 of a warp each copy one of the warp's eight rows of tile t into ring stage `dst`.
GB_DEVINL void issue_task(const GemvParams& p, const Tile& t, int warp, int lane, uint8_t* dst, uint64_t* bar) {
  const int nsb_slice = min(p.sb_per_slice, p.n_sb - t.slice * p.sb_per_slice);
  const int nsb = min(p.sb_per_chunk, nsb_slice - t.chunk * p.sb_per_chunk);
  int64_t row;
  const uint8_t* src = lane < 8 ? tile_row_ptr(p, t, warp, lane, &row) : nullptr;
  uint32_t bytes = 0, head = 0;
  if (src) {
    head = (uint32_t)((uintptr_t)src & 15u);
    bytes = (head + (uint32_t)nsb * (uint32_t)p.fmt.type_size + 15u) & ~15u;
  }
  uint32_t total = bytes;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) gb_mbar_expect_tx(bar, total);     // total == 0 completes the phase at once
  __syncwarp();
  if (src) gb_bulk_g2s(dst + lane * p.row_pitch, src - head, bytes, bar);
}

template <int kFmt, bool kMoE, bool kWide, bool kLit>
__global__ void __launch_bounds__(kLit ? 512 : 256, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
  const int kThreads = blockDim.x;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);             // [warps][kMaxStages]
  uint16_t* sub_tab = reinterpret_cast<uint16_t*>(smem + 512);        // 16 bf16 two-tier multipliers
  int* xsrc_s = reinterpret_cast<int*>(smem + 576);                   // routed: source rows of the staged pass (<= 16)
  int* tile_base_s = reinterpret_cast<int*>(smem + 1280);             // routed: [E + 1] tile prefix, [E + 1] offsets
  int* offs_s = tile_base_s + (p.E + 1);
  uint8_t* lut = smem + 1280 + p.etab_bytes;
  uint8_t* xs = lut + p.lut_bytes;
  uint8_t* rings = xs + p.x_rows * p.x_pitch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool fp8 = (kFmt == kFp8Prod4 || kFmt == kFp8Prod2);

  if (tid == 0) {
    for (int s = 0; s < kMaxWarps * kMaxStages; ++s) gb_mbar_init(&full_bar[s], 1);
    gb_fence_barrier_init();
  }
  if (tid < 16 && p.fmt.scale_coding == GB_SCALE_V2)
    sub_tab[tid] = (uint16_t)(__float_as_uint(p.compose[127 * 16 + tid]) >> 16);   // T[c], exact in bf16
  gb_pdl_launch_dependents();
  if constexpr (kMoE) {
    gb_pdl_wait();                     // the routing tables come from the kernel before
    // Every CTA walks the same global tile list; build its per-expert prefix once, in shared
    // memory, so that finding a tile is a short search instead of a pass over all experts.
    for (int e = tid; e <= p.E; e += kThreads) offs_s[e] = p.offsets[e];
    __syncthreads();
    if (warp == 0) {
      int running = 0;
      for (int base = 0; base < p.E; base += 32) {
        const int e = base + lane;
        const int cnt = e < p.E ? offs_s[e + 1] - offs_s[e] : 0;
        const int v = ((cnt + p.m_chunk - 1) / p.m_chunk) * p.n_row_tiles;
        int incl = v;
#pragma unroll
        for (int dd = 1; dd < 32; dd <<= 1) {
          const int n = __shfl_up_sync(0xffffffffu, incl, dd);
          if (lane >= dd) incl += n;
        }
        if (e < p.E) tile_base_s[e] = running + incl - v;
        running += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) tile_base_s[p.E] = running;
    }
  }
  __syncthreads();

  const int g = lane >> 2, t4 = lane & 3;
  LaneDecode d;
  {
    d.bit0 = (uint32_t)t4 * (uint32_t)p.fmt.k_bits;
    d.kstep = 4u * (uint32_t)p.fmt.k_bits;
    d.scale_off = 4u * p.fmt.k_bits;
    d.ent_shift = p.lut_rep > 1 ? 7u : 4u;
    d.rep_off = p.lut_rep > 1 ? ((uint32_t)lane & 7u) << 4 : 0u;
    const bool product = p.fmt.mode == GB_MODE_PRODUCT;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      d.mask[i] = product ? ((1u << p.split.width[i]) - 1u) : 0u;
      d.shift[i] = product ? (uint32_t)p.split.shift[i] : 0u;
      d.lbase[i] = product ? (uint32_t)p.split.base[i] * 2u : 0u;
    }
    if (!product) d.mask[0] = p.fmt.k_bits >= 32 ? 0xFFFFFFFFu : ((1u << p.fmt.k_bits) - 1u);
  }
  const uint32_t lut_s = gb_smem_u32(lut), xs_s = gb_smem_u32(xs), sub_s = gb_smem_u32(sub_tab);
  // literal layout: byte selectors (index byte t4; scale byte 2(kb&1) + (t4>>1), duplicated into both halves)
  const uint32_t sel_idx = 0x4440u | (uint32_t)t4;
  const uint32_t sel_sc_even = 0x4040u | ((uint32_t)t4 >> 1) | (((uint32_t)t4 >> 1) << 8);
  const uint32_t sel_sc_odd = 0x4040u | (2u + ((uint32_t)t4 >> 1)) | ((2u + ((uint32_t)t4 >> 1)) << 8);
  uint8_t* my_ring = rings + (size_t)warp * p.stages * p.stage_bytes;
  const uint32_t ring_s = gb_smem_u32(my_ring);
  uint64_t* my_bar = full_bar + warp * kMaxStages;
  const uint32_t lut_lane = lut_s + d.rep_off;      // literal path: eight copies of every entry, pitch 128
  const uint32_t ts = (uint32_t)p.fmt.type_size;
  const bool v1 = p.fmt.scale_coding == GB_SCALE_V1;

  // ---- fill this warp's ring: the weight stream does not depend on the activations ----
  TileWalker<kMoE> ahead(p, tile_base_s, offs_s);
  Tile ta;
  bool more = true;
  for (int i = 0; i < p.stages; ++i) {
    more = more && ahead.next(ta);
    if (more) issue_task(p, ta, warp, lane, my_ring + (size_t)i * p.stage_bytes, &my_bar[i]);
  }

  // Dense: everything above read weights and constants only, and ran alongside the tail of
  // the kernel before; the activations and the outputs are touched from here on.
  if constexpr (!kMoE) gb_pdl_wait();

  int64_t lut_off = -1;
  int x_expert = -1, x_m0 = -1, cur_slice = -1;
  TileWalker<kMoE> walk(p, tile_base_s, offs_s);
  Tile t;
  float acc0[4], acc1[4];
  float accx[6][4];              // further independent chains: an MMA result is ~30 cycles away
  for (int it = 0; walk.next(t); ++it) {
    const int s = it % p.stages;
    const int sb0 = t.slice * p.sb_per_slice;
    const int nsb_slice = min(p.sb_per_slice, p.n_sb - sb0);
    const int nsb = min(p.sb_per_chunk, nsb_slice - t.chunk * p.sb_per_chunk);   // superblocks of this step

    // ---- this lane's row, and the codebook block(s) of the task's rows ----
    int64_t out_row;
    const uint8_t* my_src = tile_row_ptr(p, t, warp, g, &out_row);
    const bool row_ok = my_src != nullptr;
    int64_t off_lo = 0, my_cb_off = 0;
    bool uniform = true;            // per warp: do my eight rows share the staged codebook block?
    if (p.cb_row_offset) {
      off_lo = p.cb_row_offset[t.row0];
      if (row_ok) my_cb_off = p.cb_row_offset[out_row];
      uniform = __all_sync(0xffffffffu, !row_ok || my_cb_off == off_lo);
    }
    bool restage_x;
    if constexpr (kMoE) restage_x = (t.expert != x_expert) || (t.m0 != x_m0);
    else restage_x = (t.slice != cur_slice);
    const bool restage_lut = off_lo != lut_off;       // same verdict in every warp of the CTA
    if (restage_x || restage_lut) {
      if (it > 0) __syncthreads();     // everyone is done with the previous contents
      if (restage_lut) {
        stage_lut<kFmt>(p, lut, off_lo, tid, kThreads);
        lut_off = off_lo;
      }
      if (restage_x) {
        const int vec_per_row = nsb_slice * 32;     // 16-byte vectors of this K slice
        if constexpr (kMoE) {
          // the pass's source rows first (two dependent global loads each), so that the copy
          // loop below is one independent load per vector
          if (tid < t.mcount) {
            const int pair = p.order[t.m0 + tid];
            xsrc_s[tid] = p.x_row ? p.x_row[pair] : pair;
          }
          __syncthreads();
        }
#pragma unroll 4
        for (int i = tid; i < t.mcount * vec_per_row; i += kThreads) {
          const int m = i / vec_per_row, v = i - m * vec_per_row;
          int64_t src_row = m;
          if constexpr (kMoE) src_row = xsrc_s[m];
          uint4 val = *reinterpret_cast<const uint4*>(p.x + src_row * p.K + (int64_t)sb0 * 256 + v * 8);
          // fused bucket: a group of 16 is this lane's vector and its neighbour's (whole warps
          // enter the loop together: the vector count is a multiple of 32)
          if (p.act == GB_ACT_FP4_GROUP16) val = gb_fp4_group16_qdq_pair(val, p.scale_rule);
          *reinterpret_cast<uint4*>(xs + m * p.x_pitch + v * 16) = val;
        }
        if constexpr (kMoE) { x_expert = t.expert; x_m0 = t.m0; }
        else cur_slice = t.slice;
      }
      __syncthreads();
    }

    // A wait that runs out raises the status word and carries on (the output is then
    // garbage, and flagged): leaving here would strand the other warps at a CTA barrier.
    uint32_t tok;
    if (!gb_mbar_wait(&my_bar[s], (it / p.stages) & 1, &tok)) atomicExch(p.status, 2);
    uint32_t sbp = ring_s + (uint32_t)s * (uint32_t)p.stage_bytes + (uint32_t)g * (uint32_t)p.row_pitch +
                   (row_ok ? (uint32_t)((uintptr_t)my_src & 15u) : 0u);
    const uint32_t warp_head = __shfl_sync(0xffffffffu, (uint32_t)((uintptr_t)my_src & 15u), 0);
    // fp8 grid: the served weight is bf16(value * row scale), rounded per weight
    float row_scale = 1.0f;
    if constexpr (fp8) {
      if (row_ok) row_scale = p.weight_scale[(int64_t)t.expert * p.N + out_row];
    }

    if (t.chunk == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc0[i] = 0.f; acc1[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 6; ++j) accx[j][i] = 0.f;
      }
    }
    // MMA rows without an activation row this pass re-read the last live row (a broadcast,
    // no extra shared-memory traffic): their output rows are simply never stored.  Lanes whose
    // weight row lies past the edge decode the task's first row, likewise unused.  The loop
    // below is branch-free.
    const uint32_t x_lane = (uint32_t)t4 * 16u;
    const uint32_t x_chunk = (uint32_t)(t.chunk * p.sb_per_chunk) * 512u;
    uint32_t xa_s = xs_s + (uint32_t)min(g, t.mcount - 1) * (uint32_t)p.x_pitch + x_lane + x_chunk;
    uint32_t xb_s = xs_s + (uint32_t)min(g + 8, t.mcount - 1) * (uint32_t)p.x_pitch + x_lane + x_chunk;
    const uint32_t xa_step = 512u, xb_step = 512u;
    if (!row_ok) sbp = ring_s + (uint32_t)s * (uint32_t)p.stage_bytes + warp_head;

    if (uniform) {
      // Software-pipelined by superblock: all shared-memory reads of a superblock (codes,
      // table entries, scales, activations) are issued together, so a warp pays one
      // shared-memory round trip per 256 weights instead of one per 32.
      const bool hi_any = t.mcount > 8;          // uniform: any activation row in MMA rows 8..15
      for (int sb = 0; sb < nsb; ++sb, sbp += ts, xa_s += xa_step, xb_s += xb_step) {
        uint32_t w[8][4], s2[8];
        uint4 xa[8];
        if constexpr (kLit) {
          const uint4 iw0 = ldt_v4(sbp, tok), iw1 = ldt_v4(sbp + 16, tok), sw = ldt_v4(sbp + 32, tok);
          const uint32_t iw[8] = {iw0.x, iw0.y, iw0.z, iw0.w, iw1.x, iw1.y, iw1.z, iw1.w};
          const uint32_t scw[4] = {sw.x, sw.y, sw.z, sw.w};
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) {
            const uint4 v = ldt_v4(lut_lane + (__byte_perm(iw[kb], 0u, sel_idx) << 7), tok);
            w[kb][0] = v.x; w[kb][1] = v.y; w[kb][2] = v.z; w[kb][3] = v.w;
          }
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) xa[kb] = ldt_v4(xa_s + kb * 64, tok);
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) {
            const uint32_t b2 = __byte_perm(scw[kb >> 1], 0u, (kb & 1) ? sel_sc_odd : sel_sc_even);
            s2[kb] = ((b2 & 0x007F007Fu) << 4) | ((b2 & 0x00800080u) << 8);      // scale * 2^-120, both halves
          }
        } else {
          uint32_t lo[8], hi[8], sraw[8];
          uint32_t super_bits = 0;
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) fetch_code<kWide>(sbp, d.bit0 + kb * d.kstep, lo[kb], hi[kb]);
          if constexpr (!fp8) {
            // group (4 kb + t4) / 2 = 2 kb + (t4 >> 1)
            if (v1) {
#pragma unroll
              for (int kb = 0; kb < 8; ++kb) sraw[kb] = lds_u8(sbp + d.scale_off + 2u * kb + ((uint32_t)t4 >> 1));
            } else {
              super_bits = (lds_u8(sbp + d.scale_off) - 127u) << 7;               // two-tier exponent, once
#pragma unroll
              for (int kb = 0; kb < 8; ++kb) sraw[kb] = lds_u8(sbp + d.scale_off + 1u + kb);   // groups 2kb, 2kb+1
            }
          }
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) expand_code<kFmt, kWide>(d, lut_s, lo[kb], hi[kb], w[kb]);
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) xa[kb] = ldt_v4(xa_s + kb * 64, tok);
          if constexpr (!fp8) {
            if (v1) {
#pragma unroll
              for (int kb = 0; kb < 8; ++kb)
                s2[kb] = (((sraw[kb] & 0x7Fu) << 4) | ((sraw[kb] & 0x80u) << 8)) * 0x10001u;   // scale * 2^-120
            } else {
              uint32_t tb[8];
#pragma unroll
              for (int kb = 0; kb < 8; ++kb)
                tb[kb] = lds_u16(sub_s + ((sraw[kb] >> (((uint32_t)t4 >> 1) * 4u)) & 0xFu) * 2u);
#pragma unroll
              for (int kb = 0; kb < 8; ++kb) s2[kb] = ((tb[kb] + super_bits) & 0xFFFFu) * 0x10001u;   // T[c] 2^(E-127)
            }
          }
        }
#pragma unroll
        for (int kb = 0; kb < 8; ++kb) {
          // k-block kb = weights [32 kb, 32 kb + 32): this lane holds codeword 4 kb + t4
          if constexpr (fp8) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float flo = __uint_as_float(w[kb][j] << 16) * row_scale;
              const float fhi = __uint_as_float(w[kb][j] & 0xFFFF0000u) * row_scale;
              asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[kb][j]) : "f"(fhi), "f"(flo));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) w[kb][j] = mul_bf16x2(w[kb][j], s2[kb]);
          }
          uint4 xb = xa[kb];                     // M <= 8: rows 8..15 mirror rows 0..7, unused
          if (hi_any) xb = ldt_v4(xb_s + kb * 64, tok);
          const uint32_t a0[4] = {xa[kb].x, xb.x, xa[kb].y, xb.y};
          const uint32_t a1[4] = {xa[kb].z, xb.z, xa[kb].w, xb.w};
          if ((kb & 3) == 0) {
            gb_mma_bf16_16816(acc0, a0, w[kb][0], w[kb][1]);
            gb_mma_bf16_16816(acc1, a1, w[kb][2], w[kb][3]);
          } else {
            gb_mma_bf16_16816(accx[2 * (kb & 3) - 2], a0, w[kb][0], w[kb][1]);
            gb_mma_bf16_16816(accx[2 * (kb & 3) - 1], a1, w[kb][2], w[kb][3]);
          }
        }
      }
    } else {
      mixed_codebook_task<fp8>(p, d, sbp, nsb, my_cb_off, row_scale, xa_s, xb_s, xa_step, xb_step, sub_s, t4,
                               acc0, acc1);
    }
    // ---- the stage is free: refill it with the task kMaxStages ahead ----
    __syncwarp();
    more = more && ahead.next(ta);
    if (more) issue_task(p, ta, warp, lane, my_ring + (size_t)s * p.stage_bytes, &my_bar[s]);

    if (t.chunk + 1 < t.nchunks) continue;          // more K chunks of this tile to come

    // ---- results: lane (g, t4) holds C[m = g (+8)][n = 2 t4 (+1)], n = row inside the task ----
    float c[4], raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      raw[i] = (acc0[i] + acc1[i]) + (accx[0][i] + accx[1][i]) + (accx[2][i] + accx[3][i]) + (accx[4][i] + accx[5][i]);
      c[i] = raw[i] * p.global_scale;
    }
    if (p.swiglu) {
      // rows 0..3 of the task are gate rows, 4..7 the matching up rows held two lanes on
      float up[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) up[i] = __shfl_down_sync(0xffffffffu, c[i], 2);
      if (t4 < 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = g + (i >> 1) * 8, n = 2 * t4 + (i & 1);
          if (m < t.mcount && 4 * warp + n < t.nrows) {
            const float gate = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(c[i]));
            const float upv = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(up[i]));
            const float sl = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(gate / (1.0f + __expf(-gate))));
            const int pair = p.order[t.m0 + m];
            p.y[(int64_t)pair * (p.N / 2) + t.row0 + 4 * warp + n] = (uint16_t)gb_f32_to_bf16_bits(sl * upv);
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = g + (i >> 1) * 8, n = 2 * t4 + (i & 1);
        if (m < t.mcount && 8 * warp + n < t.nrows) {
          const int64_t row = (int64_t)t.row0 + 8 * warp + n;
          if (p.ksplit > 1) {
            atomicAdd(p.ws + (int64_t)m * p.N + row, raw[i]);
          } else {
            int64_t orow = m;
            uint16_t* ybase = p.y;
            if constexpr (kMoE) {
              orow = p.order[t.m0 + m];
              if (p.pairs_per_rank > 0) {       // the pair's home rank keeps its row (peer store)
                const int home = (int)(orow / p.pairs_per_rank);
                ybase = p.y_peer[home];
                orow -= (int64_t)home * p.pairs_per_rank;
              }
            }
            ybase[orow * p.N + row] = (uint16_t)gb_f32_to_bf16_bits(c[i]);
          }
        }
      }
    }
  }
}

__global__ void gemv_finalize_kernel(const float* __restrict__ ws, float global_scale,
                                     uint16_t* __restrict__ y, int64_t total) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) y[i] = (uint16_t)gb_f32_to_bf16_bits(ws[i] * global_scale);
}

using KernelFn = void (*)(const GemvParams);

template <bool kMoE>
KernelFn kernel_of(int fmt, bool wide, bool lit) {
  switch (fmt) {
    case kFp4Prod2: return gemv_kernel<kFp4Prod2, kMoE, false, false>;
    case kFp4Signed: return gemv_kernel<kFp4Signed, kMoE, false, false>;
    case kFp4Full: return lit ? gemv_kernel<kFp4Full, kMoE, false, true> : gemv_kernel<kFp4Full, kMoE, false, false>;
    case kFp8Prod4: return wide ? gemv_kernel<kFp8Prod4, kMoE, true, false> : gemv_kernel<kFp8Prod4, kMoE, false, false>;
    default: return gemv_kernel<kFp8Prod2, kMoE, false, false>;
  }
}

KernelFn pick_kernel(int fmt, bool moe, bool wide, bool lit) {
  return moe ? kernel_of<true>(fmt, wide, lit) : kernel_of<false>(fmt, wide, lit);
}

// The 48-byte literal superblock (full mode, k = 8, E4M3-direct scales) with every row slice
// on a 16-byte boundary can be read with three vector loads per superblock.
bool literal_aligned(const GemvParams& p) {
  return p.fmt.grid == GB_GRID_FP4 && p.fmt.mode == GB_MODE_FULL && p.fmt.k_bits == 8 &&
         p.fmt.scale_coding == GB_SCALE_V1 && ((uintptr_t)p.qw & 15u) == 0 && p.row_stride % 16 == 0 &&
         p.expert_stride % 16 == 0;
}

constexpr int kDotRowsMax = 8;      // most activation rows ever served by per-row table GEMVs
// Row counts at which gb_gemv changes kernel for the literal format, as measured on the
// benchmark's projections: up to four rows one table GEMV per row (weights re-streamed, mostly
// out of L2) beats expanding every weight; from seventeen rows on the tensor-core decode kernel
// (flat in the row count: gate_up 86 us at 2..16 rows, 110 us at 128) passes the expanding one.
// gb_set_row_routes moves them (a process-wide setting, meant for tests and for tuning).
std::atomic<int> g_dot_rows_max{4}, g_umma_min_rows{5};
int umma_min_rows() { return g_umma_min_rows.load(std::memory_order_relaxed); }
int dot_rows_max() { return g_dot_rows_max.load(std::memory_order_relaxed); }

int classify(const gb_format& f, int* out, bool* wide) {
  *wide = f.k_bits > 32;
  if (f.grid == GB_GRID_FP4) {
    if (f.k_bits > 32) return gb_fail(GB_EUNSUPPORTED, "fp4 grid codewords wider than 32 bits");
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 2) { *out = kFp4Prod2; return GB_OK; }
    if (f.mode == GB_MODE_SIGNED) { *out = kFp4Signed; return GB_OK; }
    if (f.mode == GB_MODE_FULL) { *out = kFp4Full; return GB_OK; }
  } else {
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 4) { *out = kFp8Prod4; return GB_OK; }
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 2 && f.k_bits <= 28) { *out = kFp8Prod2; return GB_OK; }
  }
  return gb_fail(GB_EUNSUPPORTED, "no decode-batch kernel for grid %d mode %d n_sub %d k %d", f.grid, f.mode,
                 f.n_sub, f.k_bits);
}

// Fill the tiling fields.  m_rows = activation rows a tile multiplies at once; `sms` sizes
// the K slicing of the dense case so that the tiles cover the machine.
int plan(GemvParams& p, int m_rows, bool moe, int sms, size_t* smem_bytes) {
  p.n_sb = (int)(p.K / 256);
  p.warps = literal_aligned(p) ? 16 : 8;
  const int tile_rows = 8 * p.warps;
  p.split = gb_make_split(p.fmt.k_bits, p.fmt.mode == GB_MODE_PRODUCT ? p.fmt.n_sub : 1);
  p.cb_elems = (int)gb_codebook_elems(p.fmt);
  // The literal fast path keeps eight copies of every 16-byte entry (lane l reads copy l % 8), so
  // a quarter-warp's eight lookups never collide on a bank: 4 wavefronts per lookup instead of ~10.
  p.lut_rep = literal_aligned(p) ? 8 : 1;
  p.lut_bytes = (p.cb_elems * 2 * p.lut_rep + 127) & ~127;
  if (p.lut_bytes > 72 * 1024)
    return gb_fail(GB_EUNSUPPORTED, "codebook of %d entries does not fit the shared-memory table", p.cb_elems);
  p.x_rows = m_rows;
  const int half = p.swiglu ? tile_rows / 2 : tile_rows;
  const int64_t rows_out = p.swiglu ? p.N / 2 : p.N;
  p.n_row_tiles = (int)((rows_out + half - 1) / half);
  // K slices (partial sums added atomically): (a) the staged activation rows must fit their
  // budget, (b) dense only: enough tiles to cover the SMs.
  int want = 1;
  while ((int64_t)p.x_rows * (((p.n_sb + want - 1) / want) * 512 + 64) > kXBudget) ++want;
  if (!moe) {
    while (2 * p.n_row_tiles * want < 3 * sms && want < p.n_sb && (p.n_sb + want) / (want + 1) >= 2) ++want;
  } else if (want > 1) {
    return gb_fail(GB_EUNSUPPORTED, "K=%lld is too wide for the routed decode kernel at %d rows per pass",
                   (long long)p.K, m_rows);
  }
  p.sb_per_slice = (p.n_sb + want - 1) / want;
  p.ksplit = (p.n_sb + p.sb_per_slice - 1) / p.sb_per_slice;
  p.x_pitch = p.sb_per_slice * 512 + 64;
  // Ring geometry.  A stage holds one K chunk of a warp's eight rows: per row the chunk's
  // bytes plus the alignment head and a tail the word-wise extraction may touch, on a pitch
  // that is 16 mod 32 so the eight rows start in different banks.  The chunk is the largest
  // that leaves every warp two stages (up to kMaxStages when there is room).
  p.etab_bytes = moe ? (int)((2 * (p.E + 1) * sizeof(int) + 127) & ~127ull) : 0;
  const int64_t fixed = 1280 + p.etab_bytes + p.lut_bytes + (int64_t)p.x_rows * p.x_pitch;
  const int64_t per_warp = (kSmemBig - fixed) / p.warps;
  auto pitch_of = [&](int nsb) { return (int)((((int64_t)nsb * p.fmt.type_size + 15 + 16 + 31) & ~31ll) + 16); };
  auto stage_of = [&](int nsb) { return (8 * pitch_of(nsb) + 127) & ~127; };
  int chunk = p.sb_per_slice;
  // Two stages are enough to keep a copy in flight while a stage is consumed; beyond that a
  // bigger chunk (fewer steps, each with its walk / issue / wait overhead) is worth more than depth.
  while (chunk > 1 && (int64_t)2 * stage_of(chunk) > per_warp) --chunk;
  int stages = (int)(per_warp / stage_of(chunk));
  if (stages < 2)
    return gb_fail(GB_EUNSUPPORTED, "a one-superblock stage of %d bytes leaves no room for a two-stage ring "
                   "(fixed %lld bytes)", stage_of(chunk), (long long)fixed);
  p.sb_per_chunk = chunk;
  p.row_pitch = pitch_of(chunk);
  p.stage_bytes = stage_of(chunk);
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  *smem_bytes = (size_t)(fixed + (int64_t)p.warps * p.stages * p.stage_bytes);
  return GB_OK;
}

void fill_weight(GemvParams& p, const gb_weight* w) {
  p.qw = w->qw;
  p.row_stride = w->row_stride;
  p.codebook = w->codebook;
  p.cb_row_offset = w->cb_row_offset;
  p.compose = w->compose;
  p.weight_scale = w->weight_scale;
  p.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  p.N = w->rows;
  p.K = w->K;
  p.fmt = w->fmt;
}

}  // namespace

int gb_prepare_kernels() {
  for (int f = 0; f < kNumFmt; ++f)
    for (int moe = 0; moe < 2; ++moe)
      for (int wide = 0; wide < 2; ++wide)
        for (int lit = 0; lit < 2; ++lit)
          GB_CUDA_OK(cudaFuncSetAttribute((const void*)pick_kernel(f, moe != 0, wide != 0, lit != 0),
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBig + 4096));
  return GB_OK;
}

extern "C" {

// Room for the bucketed activations (fused `act`) plus the fp32 partial sums of a
// K-sliced launch; an upper bound, valid for every format.
int64_t gb_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  const int64_t mma_path = ((M * K * 2 + 255) & ~255ll) + M * N * (int64_t)sizeof(float);
  const int64_t dot_path = gb_gemv_dot_workspace_bytes(N, K);     // M = 1, literal format
  const int64_t rows_path = gb_gemv_dot_rows_workspace_bytes(M < dot_rows_max() ? M : dot_rows_max(), N, K);   // rows 2..dot_rows_max()
  const int64_t umma_path = gb_gemv_umma_workspace_bytes(M, N, K);   // rows 2..128, literal format
  int64_t need = mma_path > dot_path ? mma_path : dot_path;
  if (umma_path > need) need = umma_path;
  return need > rows_path ? need : rows_path;
}

int gb_gemv_row_batch_max(const gb_weight* w) {
  if (gb_check_weight(w) != GB_OK) return 0;
  const int m = gb_gemv_umma_max_rows(w);
  return m > 16 ? m : 16;
}

int gb_gemv(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y,
            void* workspace, int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(x && y, "null activation or output pointer");
  GB_REQUIRE(M >= 1 && M <= 128, "decode-batch kernels take 1..128 rows, got M=%lld", (long long)M);
  GB_REQUIRE(act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16 || act == GB_ACT_FP8_TOKEN, "unknown act %d", act);
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  if (M >= umma_min_rows() || (umma_min_rows() <= 128 && !gb_gemv_umma_is_literal(w))) {
    // decode into tensor memory, tensor-core MMA with the weights on the M side; every weight is
    // decoded once whatever the row count.  The literal format has faster table kernels for a few
    // rows; the product formats it serves (padded two-tier k = 16, fp8 k = 32 and k = 16) take it from
    // one row on.  A threshold past 128 switches the kernel off for every format.
    rc = gb_gemv_umma(x, M, w, act, scale_rule, y, workspace, workspace_bytes, stream_);
    if (rc != GB_EUNSUPPORTED) return rc;
  }
  if (M > 16)
    return gb_fail(GB_EUNSUPPORTED,
                   "more than 16 rows (M=%lld) are served up to gb_gemv_row_batch_max() rows, for the formats and layouts "
                   "of the tensor-core decode kernel only",
                   (long long)M);
  if (M == 1) {
    // one activation row of the literal format: inner-product tables instead of per-weight expansion
    rc = gb_gemv_dot(x, w, act, scale_rule, y, workspace, workspace_bytes, stream_);
    if (rc != GB_EUNSUPPORTED) return rc;
  } else if (M <= dot_rows_max()) {
    // a few rows of the literal format: one table GEMV per row beats expanding every weight
    rc = gb_gemv_dot_rows(x, M, w, act, scale_rule, y, workspace, workspace_bytes, stream_);
    if (rc != GB_EUNSUPPORTED) return rc;
  }
  int fmt;
  bool wide;
  rc = classify(w->fmt, &fmt, &wide);
  if (rc != GB_OK) return rc;

  GemvParams p = {};
  fill_weight(p, w);
  p.M = (int)M;
  p.E = 1;
  p.m_chunk = 16;
  p.status = gb_status_word();
  size_t smem = 0;
  rc = plan(p, (int)M, false, sms, &smem);
  if (rc != GB_OK) return rc;

  const uint16_t* xin = (const uint16_t*)x;
  const int64_t xq_bytes = act == GB_ACT_NONE ? 0 : ((M * w->K * 2 + 255) & ~255ll);
  const int64_t ws_bytes = p.ksplit > 1 ? M * w->rows * 4 : 0;
  if (xq_bytes + ws_bytes > 0) {
    GB_REQUIRE(workspace != nullptr && workspace_bytes >= xq_bytes + ws_bytes,
               "workspace of %lld bytes is too small (need %lld)", (long long)workspace_bytes,
               (long long)(xq_bytes + ws_bytes));
  }
  if (act != GB_ACT_NONE) {
    void* xq = workspace;
    rc = act == GB_ACT_FP4_GROUP16 ? gb_fp4_act_qdq(x, xq, M, w->K, scale_rule, stream_)
                                   : gb_fp8_act_qdq(x, xq, M, w->K, scale_rule, stream_);
    if (rc != GB_OK) return rc;
    xin = (const uint16_t*)xq;
  }
  p.x = xin;
  p.y = (uint16_t*)y;
  if (p.ksplit > 1) {
    p.ws = (float*)((uint8_t*)workspace + xq_bytes);
    GB_CUDA_OK(cudaMemsetAsync(p.ws, 0, (size_t)ws_bytes, stream));
  }
  int grid = sms;
  const int tiles = p.n_row_tiles * p.ksplit;
  if (grid > tiles) grid = tiles;
  grid = (grid / p.ksplit) * p.ksplit;
  if (grid < p.ksplit) grid = p.ksplit;
  GB_CUDA_OK(gb_launch(pick_kernel(fmt, false, wide, literal_aligned(p)), dim3(grid), dim3(32 * p.warps), smem, stream, p));
  if (p.ksplit > 1) {
    const int64_t total = M * w->rows;
    GB_CUDA_OK(gb_launch(gemv_finalize_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                         (const float*)p.ws, p.global_scale, p.y, total));
  }
  return GB_OK;
}

int64_t gb_moe_gemv_workspace_bytes(int64_t P, int64_t rows) {
  (void)P; (void)rows;
  return 0;
}

int gb_moe_gemv(const void* x, const int32_t* x_row, const gb_weight* w, int64_t expert_stride,
                int64_t E, const int32_t* offsets, const int32_t* order, int64_t P, int swiglu,
                int act, int scale_rule, void* y, const gb_peer_rows* y_rows, void* workspace,
                int64_t workspace_bytes, void* stream_) {
  (void)workspace; (void)workspace_bytes;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(x && (y || y_rows) && offsets && order, "null pointer argument");
  GB_REQUIRE(!(y_rows && swiglu), "per-rank output rows are for the down projection, not the fused gate/up");
  GB_REQUIRE(E >= 1 && P >= 0, "bad E=%lld P=%lld", (long long)E, (long long)P);
  GB_REQUIRE(!swiglu || w->rows % 2 == 0, "swiglu needs an even row count");
  GB_REQUIRE(act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16,
             "the routed kernel fuses the fp4 group-16 bucket only (act %d)", act);
  if (P == 0) return GB_OK;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  int fmt;
  bool wide;
  rc = classify(w->fmt, &fmt, &wide);
  if (rc != GB_OK) return rc;

  GemvParams p = {};
  fill_weight(p, w);
  p.x = (const uint16_t*)x;
  p.x_row = x_row;
  p.expert_stride = expert_stride;
  p.offsets = offsets;
  p.order = order;
  p.E = (int)E;
  p.swiglu = swiglu ? 1 : 0;
  p.act = act;
  p.scale_rule = scale_rule;
  p.y = (uint16_t*)y;
  if (y_rows) {
    GB_REQUIRE(y_rows->rows_per_rank > 0 && (P + y_rows->rows_per_rank - 1) / y_rows->rows_per_rank <= 8,
               "bad per-rank output rows: %lld per rank for %lld pairs", (long long)y_rows->rows_per_rank, (long long)P);
    for (int r = 0; r * y_rows->rows_per_rank < P; ++r) {
      GB_REQUIRE(y_rows->base[r] != nullptr, "per-rank output rows: rank %d has no buffer", r);
      p.y_peer[r] = (uint16_t*)y_rows->base[r];
    }
    p.pairs_per_rank = (int)y_rows->rows_per_rank;
  }
  p.status = gb_status_word();
  // tokens per pass: as many (up to sixteen) as the activation budget holds
  const int64_t pitch = (w->K / 256) * 512 + 64;
  int mc = (int)(kXBudget / pitch);
  if (mc > 16) mc = 16;
  if (P < mc) mc = (int)P;
  if (mc < 1)
    return gb_fail(GB_EUNSUPPORTED, "K=%lld is too wide for the routed decode kernel", (long long)w->K);
  p.m_chunk = mc;
  size_t smem = 0;
  rc = plan(p, mc, true, sms, &smem);
  if (rc != GB_OK) return rc;
  GB_CUDA_OK(gb_launch(pick_kernel(fmt, true, wide, literal_aligned(p)), dim3(sms), dim3(32 * p.warps), smem, stream, p));
  return GB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// gb_gemv_static: the decode-batch linear for callers that must not allocate.
// ---------------------------------------------------------------------------
// Its scratch (bucketed activations + fp32 partial sums of a K-sliced launch) lives in
// this file-scope device array instead of a caller-provided workspace.  Every device that
// loads the library carries the array until the process exits.
__device__ __align__(256) static unsigned char g_gemv_static_scratch[GB_GEMV_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mutex;
std::atomic<void*> g_static_ptr[64];  // device address of the array, per device ordinal (null until looked up)
}  // namespace

extern "C" int gb_set_row_routes(int dot_rows, int umma_min) {
  GB_REQUIRE(dot_rows >= 0 && dot_rows <= kDotRowsMax, "per-row table GEMVs serve up to %d rows, got %d", kDotRowsMax, dot_rows);
  GB_REQUIRE(umma_min >= 0 && umma_min <= 129, "tensor-core decode threshold %d outside [0, 129]", umma_min);
  g_dot_rows_max.store(dot_rows == 0 ? 4 : dot_rows, std::memory_order_relaxed);
  g_umma_min_rows.store(umma_min == 0 ? 5 : (umma_min < 2 ? 2 : umma_min), std::memory_order_relaxed);
  return GB_OK;
}

extern "C" int gb_gemv_static(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule,
                              void* y, void* stream) {
  GB_REQUIRE(w != nullptr, "null weight descriptor");
  GB_REQUIRE(M >= 1 && M <= 16, "decode-batch kernel takes 1..16 rows, got M=%lld", (long long)M);
  const int64_t need = gb_gemv_workspace_bytes(M, w->rows, w->K);
  GB_REQUIRE(need <= (int64_t)GB_GEMV_STATIC_SCRATCH_BYTES,
             "gb_gemv_static: M=%lld N=%lld K=%lld needs %lld bytes of scratch, the built-in array holds %lld; "
             "use gb_gemv with a caller-owned workspace for this shape",
             (long long)M, (long long)w->rows, (long long)w->K, (long long)need,
             (long long)GB_GEMV_STATIC_SCRATCH_BYTES);
  int dev = -1;
  GB_CUDA_OK(cudaGetDevice(&dev));
  GB_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  void* scratch = g_static_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // Once per device, with that device current.  In host code the array's name is only a
    // handle: the address a kernel may use has to be asked for.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_ptr[dev].load(std::memory_order_relaxed) == nullptr) {
      void* p = nullptr;
      GB_CUDA_OK(cudaGetSymbolAddress(&p, g_gemv_static_scratch));
      g_static_ptr[dev].store(p, std::memory_order_release);
    }
    scratch = g_static_ptr[dev].load(std::memory_order_relaxed);
  }
  // gb_gemv overwrites the activation part and clears the partial sums it uses (an async
  // memset on the caller's stream, not an allocation) before the kernel adds into them.
  return gb_gemv(x, M, w, act, scale_rule, y, scratch, (int64_t)GB_GEMV_STATIC_SCRATCH_BYTES, stream);
}

