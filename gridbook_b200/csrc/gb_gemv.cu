// Decode-batch (M <= 16) codebook linear and grouped routed-MoE GEMV.
//
// One persistent CTA per SM walks tiles of eight output rows.  A producer warp
// streams each tile's packed rows into a shared-memory ring with 1-D bulk copies
// (16-byte aligned windows around rows of any stride, so odd type_size rows need
// no repacking); eight consumer warps split the tile's K range, expand each
// codeword through a shared-memory codebook into bf16 grid values times the
// group scale (exact: <= 6 significant bits), and feed them to m16n8k16 bf16 MMAs
// against the activation rows held in shared memory.  Partials are reduced across
// warps in shared memory, scaled and rounded to bf16 once.
#include "gb_common.cuh"

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileRows = 8;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kXBudget = 96 * 1024;

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
  int m_chunk;            // tokens per tile pass (MoE), multiple of... <= 16
  // tiling
  int ksplit, sb_per_slice, n_sb;
  int n_row_tiles;
  int stages, stage_bytes, run_pitch, piece_pitch;
  int x_pitch;            // bytes between activation rows in shared memory
  int x_rows;             // 8 or 16 rows staged
  int lut_bytes;
  // outputs
  uint16_t* y;
  float* ws;              // [M, N] fp32 partial sums when ksplit > 1
  int* status;
};

struct Tile {
  int row0;       // first output row (gate row for swiglu)
  int nrows;      // valid rows in the (half) tile
  int expert;
  int m0, mcount; // sorted-pair range of this pass (MoE) or [0, M)
  int slice;
};

// Every thread of the CTA enumerates the same tile sequence.
template <bool kMoE>
struct TileWalker {
  const GemvParams& p;
  int next_local;   // dense: next row-tile index; MoE: next global tile index for this CTA
  int e, base;      // MoE: current expert and the global index of its first tile
  __device__ explicit TileWalker(const GemvParams& pp) : p(pp) {
    if constexpr (kMoE) {
      next_local = blockIdx.x; e = 0; base = 0;
    } else {
      next_local = blockIdx.x / p.ksplit;
    }
  }
  __device__ bool next(Tile& t) {
    if constexpr (!kMoE) {
      if (next_local >= p.n_row_tiles) return false;
      t.row0 = next_local * kTileRows;
      t.nrows = min(kTileRows, (int)(p.N - t.row0));
      t.expert = 0; t.m0 = 0; t.mcount = p.M;
      t.slice = blockIdx.x % p.ksplit;
      next_local += gridDim.x / p.ksplit;
      return true;
    } else {
      const int half = p.swiglu ? kTileRows / 2 : kTileRows;
      while (e < p.E) {
        const int cnt = p.offsets[e + 1] - p.offsets[e];
        const int nch = (cnt + p.m_chunk - 1) / p.m_chunk;
        const int ntiles = nch * p.n_row_tiles;
        if (next_local < base + ntiles) {
          const int local = next_local - base;
          const int ch = local / p.n_row_tiles, rt = local - ch * p.n_row_tiles;
          const int rows_out = p.swiglu ? (int)(p.N / 2) : (int)p.N;
          t.row0 = rt * half;
          t.nrows = min(half, rows_out - t.row0);
          t.expert = e;
          t.m0 = p.offsets[e] + ch * p.m_chunk;
          t.mcount = min(p.m_chunk, cnt - ch * p.m_chunk);
          t.slice = 0;
          next_local += gridDim.x;
          return true;
        }
        base += ntiles;
        ++e;
      }
      return false;
    }
  }
};

struct StagePlan {
  int n_copies;
  const uint8_t* src[kTileRows];
  uint32_t dst[kTileRows];
  uint32_t bytes[kTileRows];
  uint32_t row_off[kTileRows];   // byte offset of row g's first superblock inside the stage
  uint32_t total;
};

// Where each row of a tile lives in global memory and in its stage buffer.
GB_DEVINL void plan_stage(const GemvParams& p, const Tile& t, StagePlan& s) {
  const uint8_t* ebase = p.qw + (int64_t)t.expert * p.expert_stride;
  const int sb0 = t.slice * p.sb_per_slice;
  const int nsb = min(p.sb_per_slice, p.n_sb - sb0);
  s.total = 0;
  if (p.ksplit == 1) {
    const int runs = p.swiglu ? 2 : 1;
    s.n_copies = runs;
    for (int r = 0; r < runs; ++r) {
      const int64_t first = (int64_t)t.row0 + (r ? p.N / 2 : 0);
      const uint8_t* a = ebase + first * p.row_stride;
      const uint32_t head = (uint32_t)((uintptr_t)a & 15u);
      const uint32_t bytes = (head + (uint32_t)t.nrows * (uint32_t)p.row_stride + 15u) & ~15u;
      s.src[r] = a - head;
      s.dst[r] = r * p.run_pitch;
      s.bytes[r] = bytes;
      s.total += bytes;
      for (int g = 0; g < t.nrows; ++g)
        s.row_off[r * (kTileRows / 2) + g] = r * p.run_pitch + head + g * (uint32_t)p.row_stride;
    }
  } else {
    s.n_copies = t.nrows;
    for (int g = 0; g < t.nrows; ++g) {
      const uint8_t* a = ebase + ((int64_t)t.row0 + g) * p.row_stride + (int64_t)sb0 * p.fmt.type_size;
      const uint32_t head = (uint32_t)((uintptr_t)a & 15u);
      const uint32_t bytes = (head + (uint32_t)nsb * p.fmt.type_size + 15u) & ~15u;
      s.src[g] = a - head;
      s.dst[g] = g * p.piece_pitch;
      s.bytes[g] = bytes;
      s.total += bytes;
      s.row_off[g] = g * p.piece_pitch + head;
    }
  }
}

GB_DEVINL void named_barrier_consumers() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}

GB_DEVINL uint32_t lds32(const uint8_t* base, uint32_t off) {
  return *reinterpret_cast<const uint32_t*>(base + off);
}

// Expand one codeword into eight bf16 grid values (four packed registers).
template <int kFmt>
GB_DEVINL void decode_codeword(const GemvParams& p, const uint8_t* lut, uint64_t code,
                               uint32_t (&w)[4]) {
  if constexpr (kFmt == kFp4Full) {
    const uint4 v = *reinterpret_cast<const uint4*>(lut + (uint32_t)code * 16u);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else if constexpr (kFmt == kFp4Signed) {
    const uint4 v = *reinterpret_cast<const uint4*>(lut + (uint32_t)(code >> 8) * 16u);
    const uint32_t s = (uint32_t)code & 0xFFu;
    // sign bit j flips coordinate j: bit 15 of the low half, bit 31 of the high half
    w[0] = v.x ^ (((s >> 0) & 1u) << 15) ^ (((s >> 1) & 1u) << 31);
    w[1] = v.y ^ (((s >> 2) & 1u) << 15) ^ (((s >> 3) & 1u) << 31);
    w[2] = v.z ^ (((s >> 4) & 1u) << 15) ^ (((s >> 5) & 1u) << 31);
    w[3] = v.w ^ (((s >> 6) & 1u) << 15) ^ (((s >> 7) & 1u) << 31);
  } else if constexpr (kFmt == kFp4Prod2 || kFmt == kFp8Prod2) {
    const uint32_t i0 = (uint32_t)code & ((1u << p.split.width[0]) - 1u);
    const uint32_t i1 = (uint32_t)(code >> p.split.width[0]);
    const uint2 a = *reinterpret_cast<const uint2*>(lut + i0 * 8u);
    const uint2 b = *reinterpret_cast<const uint2*>(lut + (uint32_t)p.split.base[1] * 2u + i1 * 8u);
    w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t idx = (uint32_t)(code >> p.split.shift[i]) & ((1u << p.split.width[i]) - 1u);
      w[i] = lds32(lut, (uint32_t)p.split.base[i] * 2u + idx * 4u);
    }
  }
}

GB_DEVINL uint32_t mul_bf16x2(uint32_t a, uint32_t s2) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(s2));
  return d;
}

// Copy one codebook block into the shared-memory table (as bf16).
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
    for (int i = tid; i < p.cb_elems; i += nthreads) dst[i] = src[i];
  }
}

template <int kFmt, bool kMoE>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty_bar = full_bar + kMaxStages;
  float* red = reinterpret_cast<float*>(smem + 256);                 // [8 warps][16][8]
  uint8_t* lut = smem + 256 + kConsumerWarps * 16 * 8 * 4;
  uint8_t* xs = lut + p.lut_bytes;
  uint8_t* stages = xs + p.x_rows * p.x_pitch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool fp8 = (kFmt == kFp8Prod4 || kFmt == kFp8Prod2);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      gb_mbar_init(&full_bar[s], 1);
      gb_mbar_init(&empty_bar[s], kConsumerWarps);
    }
    gb_fence_barrier_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      TileWalker<kMoE> walk(p);
      Tile t;
      StagePlan sp;
      for (int it = 0; walk.next(t); ++it) {
        const int s = it % p.stages;
        if (it >= p.stages && !gb_mbar_wait(&empty_bar[s], ((it / p.stages) - 1) & 1)) {
          atomicExch(p.status, 1);
          return;
        }
        plan_stage(p, t, sp);
        gb_mbar_expect_tx(&full_bar[s], sp.total);
        uint8_t* sbase = stages + (size_t)s * p.stage_bytes;
        for (int c = 0; c < sp.n_copies; ++c) gb_bulk_g2s(sbase + sp.dst[c], sp.src[c], sp.bytes[c], &full_bar[s]);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int g = lane >> 2, t4 = lane & 3;
  const int cw = 4 * warp + t4;                       // codeword of the superblock this lane expands
  const uint32_t cw_bit = (uint32_t)cw * (uint32_t)p.fmt.k_bits;
  const int grp = cw >> 1;
  const int ctid = tid, cthreads = kConsumerWarps * 32;

  // zero the activation rows that stay padding
  for (int i = ctid; i < p.x_rows * p.x_pitch / 4; i += cthreads) reinterpret_cast<uint32_t*>(xs)[i] = 0u;
  int64_t lut_off = -1;
  int x_expert = -1, x_m0 = -1;
  int cur_slice = -1;
  named_barrier_consumers();

  TileWalker<kMoE> walk(p);
  Tile t;
  StagePlan sp;
  for (int it = 0; walk.next(t); ++it) {
    const int s = it % p.stages;
    const int sb0 = t.slice * p.sb_per_slice;
    const int nsb = min(p.sb_per_slice, p.n_sb - sb0);

    // ---- (re)stage the activations this tile multiplies ----
    bool restage_x;
    if constexpr (kMoE) restage_x = (t.expert != x_expert) || (t.m0 != x_m0);
    else restage_x = (t.slice != cur_slice);
    // ---- this lane's row, and the codebook block(s) of the tile's rows ----
    const bool second_half = p.swiglu && g >= kTileRows / 2;
    const int g_local = p.swiglu ? (g & 3) : g;
    const bool row_ok = g_local < t.nrows;
    const int64_t out_row = (int64_t)t.row0 + g_local + (second_half ? p.N / 2 : 0);
    int64_t off_lo = 0, my_cb_off = 0;
    bool uniform = true;
    if (p.cb_row_offset) {
      off_lo = p.cb_row_offset[t.row0];
      if (row_ok) my_cb_off = p.cb_row_offset[out_row];
      uniform = __all_sync(0xffffffffu, !row_ok || my_cb_off == off_lo);   // same verdict in every warp
    }
    const bool restage_lut = uniform && (off_lo != lut_off);
    if (restage_x || restage_lut) {
      named_barrier_consumers();     // everyone is done with the previous contents
      if (restage_lut) {
        stage_lut<kFmt>(p, lut, off_lo, ctid, cthreads);
        lut_off = off_lo;
      }
      if (restage_x) {
        const int kw = nsb * 256;           // weights of K in this slice
        const int vec_per_row = kw / 8;     // 16-byte vectors
        const int mrows = t.mcount;
        for (int i = ctid; i < mrows * vec_per_row; i += cthreads) {
          const int m = i / vec_per_row, v = i - m * vec_per_row;
          int64_t src_row;
          if constexpr (kMoE) {
            const int pair = p.order[t.m0 + m];
            src_row = p.x_row ? p.x_row[pair] : pair;
          } else {
            src_row = m;
          }
          const uint4 val = *reinterpret_cast<const uint4*>(p.x + src_row * p.K + (int64_t)sb0 * 256 + v * 8);
          *reinterpret_cast<uint4*>(xs + m * p.x_pitch + v * 16) = val;
        }
        if constexpr (kMoE) {
          // rows beyond this pass must read as zero
          for (int i = ctid; i < (p.x_rows - mrows) * vec_per_row; i += cthreads) {
            const int m = mrows + i / vec_per_row, v = i % vec_per_row;
            *reinterpret_cast<uint4*>(xs + m * p.x_pitch + v * 16) = make_uint4(0, 0, 0, 0);
          }
          x_expert = t.expert; x_m0 = t.m0;
        } else {
          cur_slice = t.slice;
        }
      }
      named_barrier_consumers();
    }

    plan_stage(p, t, sp);
    if (!gb_mbar_wait(&full_bar[s], (it / p.stages) & 1)) {
      atomicExch(p.status, 2);
      return;
    }
    const uint8_t* sbase = stages + (size_t)s * p.stage_bytes;

    const uint8_t* rowp = sbase + sp.row_off[row_ok ? g : 0];
    // fp8 grid: the served weight is bf16(value * row scale), rounded per weight
    float row_scale = 1.0f;
    if constexpr (fp8) {
      if (row_ok) row_scale = p.weight_scale[(int64_t)t.expert * p.N + out_row];
    }

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool hi_rows = p.x_rows > 8;
    for (int sb = 0; sb < nsb; ++sb) {
      const uint8_t* sbp = rowp + sb * p.fmt.type_size;
      // activations: x[m][sb*256 + warp*32 + 8*t4 .. +8)
      const uint32_t xoff = (uint32_t)(sb * 256 + warp * 32 + t4 * 8) * 2u;
      const uint4 xa = *reinterpret_cast<const uint4*>(xs + g * p.x_pitch + xoff);
      uint4 xb = make_uint4(0, 0, 0, 0);
      if (hi_rows) xb = *reinterpret_cast<const uint4*>(xs + (g + 8) * p.x_pitch + xoff);

      uint32_t w[4] = {0u, 0u, 0u, 0u};
      if (row_ok) {
        // codeword bits: aligned 32-bit words around an arbitrary byte address
        const uint32_t byte_addr = (uint32_t)(uintptr_t)(sbp) + (cw_bit >> 3);
        const uint32_t mis = byte_addr & 3u;
        const uint32_t* words = reinterpret_cast<const uint32_t*>(sbp + (cw_bit >> 3) - mis);
        const uint64_t code = gb_extract_bits(words, mis * 8u + (cw_bit & 7u), p.fmt.k_bits);
        if (uniform) {
          decode_codeword<kFmt>(p, lut, code, w);
        } else {
          // rows of one tile use different codebooks: gather this row's from global memory
          const int sd = p.split.sub_dim;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            int64_t idx;
            bool neg = false;
            if (p.fmt.mode == GB_MODE_FULL) idx = (int64_t)code * 8 + j;
            else if (p.fmt.mode == GB_MODE_SIGNED) { idx = (int64_t)(code >> 8) * 8 + j; neg = (code >> j) & 1ull; }
            else {
              const int si = j / sd;
              idx = p.split.base[si] + (int64_t)((code >> p.split.shift[si]) & ((1ull << p.split.width[si]) - 1ull)) * sd + (j - si * sd);
            }
            float f;
            if constexpr (fp8) f = gb_e4m3_to_f32(reinterpret_cast<const uint8_t*>(p.codebook)[my_cb_off + idx]);
            else f = gb_bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.codebook)[my_cb_off + idx]);
            v[j] = neg ? -f : f;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            w[j] = (__float_as_uint(v[2 * j]) >> 16) | (__float_as_uint(v[2 * j + 1]) & 0xFFFF0000u);
        }
        if constexpr (fp8) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = __uint_as_float(w[j] << 16) * row_scale;
            const float hi = __uint_as_float(w[j] & 0xFFFF0000u) * row_scale;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[j]) : "f"(hi), "f"(lo));
          }
        } else {
          // group scale (exact E4M3 value) as a bf16 pair
          const uint8_t* plane = sbp + 4 * p.fmt.k_bits;
          float sc;
          if (p.fmt.scale_coding == GB_SCALE_V1) {
            sc = gb_e4m3_to_f32(plane[grp]);
          } else {
            const uint32_t e = plane[0];
            const uint32_t nib = (plane[1 + (grp >> 1)] >> ((grp & 1) * 4)) & 0xFu;
            sc = __ldg(p.compose + e * 16 + nib);
          }
          const uint32_t sb16 = __float_as_uint(sc) >> 16;
          const uint32_t s2 = sb16 | (sb16 << 16);
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = mul_bf16x2(w[j], s2);
        }
      }
      {
        const uint32_t a[4] = {xa.x, xb.x, xa.y, xb.y};
        gb_mma_bf16_16816(acc, a, w[0], w[1]);
      }
      {
        const uint32_t a[4] = {xa.z, xb.z, xa.w, xb.w};
        gb_mma_bf16_16816(acc, a, w[2], w[3]);
      }
    }
    __syncwarp();
    if (lane == 0) gb_mbar_arrive(&empty_bar[s]);

    // ---- cross-warp reduction: red[warp][m][n] ----
    float* my = red + warp * 128;
    my[g * 8 + 2 * t4] = acc[0];
    my[g * 8 + 2 * t4 + 1] = acc[1];
    my[(g + 8) * 8 + 2 * t4] = acc[2];
    my[(g + 8) * 8 + 2 * t4 + 1] = acc[3];
    named_barrier_consumers();
    if (ctid < 128) {
      const int m = ctid >> 3, n = ctid & 7;
      float v = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kConsumerWarps; ++w8) v += red[w8 * 128 + ctid];
      if (m < t.mcount) {
        if (p.swiglu) {
          // rows 0..3 are gate, 4..7 the matching up rows
          float other = 0.f;
#pragma unroll
          for (int w8 = 0; w8 < kConsumerWarps; ++w8) other += red[w8 * 128 + (ctid ^ 4)];
          if (n < 4 && n < t.nrows) {
            const int64_t grow = (int64_t)t.row0 + n, urow = grow + p.N / 2;
            const float gs = p.global_scale, us = p.global_scale;
            (void)urow;
            const float gate = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(v * gs));
            const float up = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(other * us));
            const float sl = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(gate / (1.0f + __expf(-gate))));
            const int pair = p.order[t.m0 + m];
            p.y[(int64_t)pair * (p.N / 2) + grow] = (uint16_t)gb_f32_to_bf16_bits(sl * up);
          }
        } else if (n < t.nrows) {
          const int64_t row = (int64_t)t.row0 + n;
          if (p.ksplit > 1) {
            atomicAdd(p.ws + (int64_t)m * p.N + row, v);
          } else {
            const float sc = p.global_scale;
            int64_t orow = m;
            if constexpr (kMoE) orow = p.order[t.m0 + m];
            p.y[orow * p.N + row] = (uint16_t)gb_f32_to_bf16_bits(v * sc);
          }
        }
      }
    }
    named_barrier_consumers();
  }
}

__global__ void gemv_finalize_kernel(const float* __restrict__ ws, const float* __restrict__ weight_scale,
                                     float global_scale, uint16_t* __restrict__ y, int64_t M, int64_t N) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float sc = global_scale;
  if (weight_scale) sc *= weight_scale[i % N];
  y[i] = (uint16_t)gb_f32_to_bf16_bits(ws[i] * sc);
}

using KernelFn = void (*)(const GemvParams);

KernelFn pick_kernel(int fmt, bool moe) {
  static const KernelFn dense[kNumFmt] = {gemv_kernel<kFp4Prod2, false>, gemv_kernel<kFp4Signed, false>,
                                         gemv_kernel<kFp4Full, false>, gemv_kernel<kFp8Prod4, false>,
                                         gemv_kernel<kFp8Prod2, false>};
  static const KernelFn routed[kNumFmt] = {gemv_kernel<kFp4Prod2, true>, gemv_kernel<kFp4Signed, true>,
                                          gemv_kernel<kFp4Full, true>, gemv_kernel<kFp8Prod4, true>,
                                          gemv_kernel<kFp8Prod2, true>};
  return moe ? routed[fmt] : dense[fmt];
}

int classify(const gb_format& f, int* out) {
  if (f.grid == GB_GRID_FP4) {
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 2) { *out = kFp4Prod2; return GB_OK; }
    if (f.mode == GB_MODE_SIGNED) { *out = kFp4Signed; return GB_OK; }
    if (f.mode == GB_MODE_FULL) { *out = kFp4Full; return GB_OK; }
  } else {
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 4) { *out = kFp8Prod4; return GB_OK; }
    if (f.mode == GB_MODE_PRODUCT && f.n_sub == 2) { *out = kFp8Prod2; return GB_OK; }
  }
  return gb_fail(GB_EUNSUPPORTED, "no decode-batch kernel for grid %d mode %d n_sub %d", f.grid, f.mode,
                 f.n_sub);
}

// Fill the tiling fields.  m_rows = activation rows a tile multiplies at once.
int plan(GemvParams& p, int m_rows, bool moe, size_t* smem_bytes) {
  p.n_sb = (int)(p.K / 256);
  p.split = gb_make_split(p.fmt.k_bits, p.fmt.mode == GB_MODE_PRODUCT ? p.fmt.n_sub : 1);
  p.cb_elems = (int)gb_codebook_elems(p.fmt);
  p.lut_bytes = (p.cb_elems * 2 + 127) & ~127;
  if (p.lut_bytes > 72 * 1024)
    return gb_fail(GB_EUNSUPPORTED, "codebook of %d entries does not fit the shared-memory table", p.cb_elems);
  p.x_rows = m_rows > 8 ? 16 : 8;
  // K slicing so the staged activations fit their budget
  p.ksplit = 1;
  p.sb_per_slice = p.n_sb;
  if (!moe) {
    while ((int64_t)p.x_rows * (p.sb_per_slice * 512 + 64) > kXBudget) {
      ++p.ksplit;
      p.sb_per_slice = (p.n_sb + p.ksplit - 1) / p.ksplit;
    }
    p.ksplit = (p.n_sb + p.sb_per_slice - 1) / p.sb_per_slice;
  }
  p.x_pitch = p.sb_per_slice * 512 + 64;
  const int half = p.swiglu ? kTileRows / 2 : kTileRows;
  const int64_t rows_out = p.swiglu ? p.N / 2 : p.N;
  p.n_row_tiles = (int)((rows_out + half - 1) / half);
  const int64_t slice_bytes = (int64_t)p.sb_per_slice * p.fmt.type_size;
  if (p.ksplit == 1) {
    p.run_pitch = (int)((half * p.row_stride + 15 + 15) & ~15) + 16;
    p.piece_pitch = 0;
    p.stage_bytes = (p.swiglu ? 2 : 1) * p.run_pitch + 16;
  } else {
    p.piece_pitch = (int)((slice_bytes + 15 + 15) & ~15) + 16;
    p.run_pitch = 0;
    p.stage_bytes = kTileRows * p.piece_pitch + 16;
  }
  p.stage_bytes = (p.stage_bytes + 127) & ~127;
  const int64_t fixed = 256 + kConsumerWarps * 16 * 8 * 4 + p.lut_bytes + (int64_t)p.x_rows * p.x_pitch;
  int64_t room = kSmemBudget - fixed;
  int stages = (int)(room / p.stage_bytes);
  if (stages < 2)
    return gb_fail(GB_EUNSUPPORTED, "tile of %d bytes leaves no room for a two-stage ring (fixed %lld bytes)",
                   p.stage_bytes, (long long)fixed);
  p.stages = stages > kMaxStages ? kMaxStages : stages;
  *smem_bytes = (size_t)(fixed + (int64_t)p.stages * p.stage_bytes);
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
      GB_CUDA_OK(cudaFuncSetAttribute((const void*)pick_kernel(f, moe != 0),
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 4096));
  return GB_OK;
}

extern "C" {

// Room for the bucketed activations (fused `act`) plus the fp32 partial sums of a
// K-sliced launch; an upper bound, valid for every format.
int64_t gb_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  return ((M * K * 2 + 255) & ~255ll) + M * N * (int64_t)sizeof(float);
}

int gb_gemv(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y,
            void* workspace, int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(x && y, "null activation or output pointer");
  GB_REQUIRE(M >= 1 && M <= 16, "decode-batch kernel takes 1..16 rows, got M=%lld", (long long)M);
  GB_REQUIRE(act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16 || act == GB_ACT_FP8_TOKEN, "unknown act %d", act);
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  int fmt;
  rc = classify(w->fmt, &fmt);
  if (rc != GB_OK) return rc;

  GemvParams p = {};
  fill_weight(p, w);
  p.M = (int)M;
  p.E = 1;
  p.m_chunk = 16;
  p.status = gb_status_word();
  size_t smem = 0;
  rc = plan(p, (int)M, false, &smem);
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
  pick_kernel(fmt, false)<<<grid, kThreads, smem, stream>>>(p);
  GB_LAUNCH_OK("gemv_kernel");
  if (p.ksplit > 1) {
    const int64_t total = M * w->rows;
    gemv_finalize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        p.ws, nullptr, p.global_scale, p.y, M, w->rows);
    GB_LAUNCH_OK("gemv_finalize_kernel");
  }
  return GB_OK;
}

int64_t gb_moe_gemv_workspace_bytes(int64_t P, int64_t rows) {
  (void)P; (void)rows;
  return 0;
}

int gb_moe_gemv(const void* x, const int32_t* x_row, const gb_weight* w, int64_t expert_stride,
                int64_t E, const int32_t* offsets, const int32_t* order, int64_t P, int swiglu,
                void* y, void* workspace, int64_t workspace_bytes, void* stream_) {
  (void)workspace; (void)workspace_bytes;
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(x && y && offsets && order, "null pointer argument");
  GB_REQUIRE(E >= 1 && P >= 0, "bad E=%lld P=%lld", (long long)E, (long long)P);
  GB_REQUIRE(!swiglu || w->rows % 2 == 0, "swiglu needs an even row count");
  if (P == 0) return GB_OK;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  int fmt;
  rc = classify(w->fmt, &fmt);
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
  p.y = (uint16_t*)y;
  p.status = gb_status_word();
  // tokens per pass: sixteen when their rows fit the activation budget, else eight
  const int64_t pitch = (w->K / 256) * 512 + 64;
  int mc = 16;
  if (16 * pitch > kXBudget) mc = 8;
  if (8 * pitch > kXBudget + 32 * 1024)
    return gb_fail(GB_EUNSUPPORTED, "K=%lld is too wide for the routed decode kernel", (long long)w->K);
  p.m_chunk = mc;
  size_t smem = 0;
  rc = plan(p, mc, true, &smem);
  if (rc != GB_OK) return rc;
  pick_kernel(fmt, true)<<<sms, kThreads, smem, stream>>>(p);
  GB_LAUNCH_OK("gemv_kernel (routed)");
  return GB_OK;
}

}  // extern "C"
