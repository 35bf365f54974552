// Prefill GEMM on the block-scaled FP4 tensor cores: D[M,N] = a_scale[m] * global * sum_k
// (A[m,k] * SFA[m,k/16]) * (B[n,k] * SFB[n,k/16]) with A and B packed E2M1 (two per byte, K-major)
// and UE4M3 scale factors per sixteen elements: tcgen05.mma kind::mxf4nvf4, block16, fp32
// accumulator in tensor memory.  B is the native NVFP4 view of a codebook layer written by the
// expander (gb_expand_fp4_nvfp4: 0.56 bytes per weight instead of the 2-byte bf16 tile), A the
// activations through gb_nvfp4_quantize_rows below.  Replaces the reference's block-scaled
// prefill (gridbook/csrc/cb_fused_fp4_gemm.cu:291-450,758-903) with the operands decoded once.
//
// Scale factors travel in the 128 x 4 atom layout (gridbook/codec.py:353-374): 512 bytes hold the
// scale bytes of 128 rows x 4 groups, row r and group g at (r % 32) * 16 + (r / 32) * 4 + g; the
// atoms of one 128-row tile follow each other along K.  One atom is exactly what one MMA
// (K = 64) needs for 128 rows: four columns of tensor memory, row r's four bytes at lane r % 32
// of every lane quarter, column r / 32.
//
// Persistent CTAs walk 128 x 256 output tiles, M fastest.  Warp 4 streams 256-element K slabs
// of A and B (tiled TMA, 128-byte swizzle) and their scale-factor atoms (bulk copies) into a
// four-stage ring; warps 6-9 move the atoms from shared to tensor memory (one thread per lane);
// warp 5 issues four MMAs per stage; warps 0-3 drain the accumulator.  Tensor memory: 256 accumulator columns and two sets of 16 SFA
// + 32 SFB columns - there is no room for a second accumulator beside them, so the epilogue of a
// tile only overlaps the loads of the next one.
#include "gb_common.cuh"

#include <cuda.h>

namespace {

constexpr int kBM = 128, kBN = 256;
constexpr int kSlabBytes = 128;                     // 256 E2M1 per row per stage
constexpr int kABytes = kBM * kSlabBytes;           // 16 KiB
constexpr int kBBytes = kBN * kSlabBytes;           // 32 KiB
constexpr int kSfaBytes = 4 * 512;                  // four atoms: 128 rows x 16 groups
constexpr int kSfbBytes = 2 * kSfaBytes;            // two row tiles of B
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 54 KiB
constexpr int kStages = 4;
constexpr int kTmemCols = 512;
constexpr uint32_t kAccCol = 0, kSfaCol = 256, kSfbCol = 272, kSfSet = 48;   // two sets of SF columns, used in turn
constexpr int kThreads = 320;                      // 4 epilogue warps, producer, MMA issuer, 4 scale-factor warps
constexpr int kSmem = kStages * kStageBytes + 1024 + 256;

struct Fp4Params {
  int64_t M, N, K;
  int k_tiles, m_tiles, n_tiles;
  int64_t sf_k_atoms;          // atoms along K of one row tile: K / 64
  const uint8_t* sfa;          // [ceil(M/128)][K/64][512]
  const uint8_t* sfb;          // [ceil(N/128)][K/64][512]
  const float* a_scale;        // [M] or null
  float global_scale;
  uint32_t idesc;
  uint16_t* D;
  int* status;
};

GB_DEVINL void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(gb_smem_u32(bar))
      : "memory");
}

GB_DEVINL void bulk_load(uint32_t smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(gb_smem_u32(bar)) : "memory");
}

// K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle.
GB_DEVINL uint64_t desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

GB_DEVINL void umma_fp4(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                        bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"((uint32_t)accumulate), "r"(sfa), "r"(sfb) : "memory");
}

GB_DEVINL void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(gb_smem_u32(bar)) : "memory");
}

GB_DEVINL void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (*abort_flag) return;
  if (!gb_mbar_wait(bar, parity)) {
    *abort_flag = 1;
    atomicExch(status, code);
  }
}

GB_DEVINL void tmem_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

GB_DEVINL void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}

// 32 accumulator columns of one output row -> bf16, scaled; full 16-byte stores where the row allows.
GB_DEVINL void store_chunk(const Fp4Params& p, const uint32_t (&v)[32], int64_t row, bool row_ok, float rs, int col0) {
  if (!row_ok) return;
  const int64_t ncol = p.N - col0;
  if (ncol <= 0) return;
  uint16_t* out = p.D + row * p.N + col0;
  if (ncol >= 32 && (p.N % 8) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = q * 8 + j * 2;
        w[j] = gb_pack_bf16x2(__uint_as_float(v[c]) * rs, __uint_as_float(v[c + 1]) * rs);
      }
      *reinterpret_cast<uint4*>(out + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 32; ++c)
      if (c < ncol) out[c] = (uint16_t)gb_f32_to_bf16_bits(__uint_as_float(v[c]) * rs);
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Fp4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t ring = gb_smem_u32(smem);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;
  uint64_t* acc_empty = acc_full + 1;
  uint64_t* sf_full = acc_empty + 1;                 // [2] a column set holds a stage's scale factors (four warps)
  uint64_t* sf_empty = sf_full + 2;                  // [2] the MMAs that read a column set are done (one commit)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      gb_mbar_init(&full_bar[s], 1);
      gb_mbar_init(&empty_bar[s], 1);
    }
    gb_mbar_init(acc_full, 1);
    gb_mbar_init(acc_empty, 4);
    for (int b = 0; b < 2; ++b) {
      gb_mbar_init(&sf_full[b], 4);
      gb_mbar_init(&sf_empty[b], 1);
    }
    *abort_flag = 0;
    gb_fence_barrier_init();
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(gb_smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 4) {
    // ------------------------------- producer -------------------------------
    if (lane == 0) {
      int kk = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
        const uint8_t* sfa = p.sfa + (int64_t)mt * p.sf_k_atoms * 512;
        const uint8_t* sfb0 = p.sfb + (int64_t)(2 * nt) * p.sf_k_atoms * 512;
        const bool second = (int64_t)(2 * nt + 1) * 128 < p.N;         // the tile's upper 128 columns exist
        for (int kt = 0; kt < p.k_tiles; ++kt, ++kk) {
          const int s = kk % kStages;
          wait_or_abort(&empty_bar[s], ((kk / kStages) & 1) ^ 1, abort_flag, p.status, 31);
          gb_mbar_expect_tx(&full_bar[s], second ? kStageBytes : kStageBytes - kSfaBytes);
          const uint32_t st = ring + (uint32_t)s * kStageBytes;
          tma_load_2d(st, &map_a, kt * kSlabBytes, mt * kBM, &full_bar[s]);
          tma_load_2d(st + kABytes, &map_b, kt * kSlabBytes, nt * kBN, &full_bar[s]);
          bulk_load(st + kABytes + kBBytes, sfa + (int64_t)kt * kSfaBytes, kSfaBytes, &full_bar[s]);
          bulk_load(st + kABytes + kBBytes + kSfaBytes, sfb0 + (int64_t)kt * kSfaBytes, kSfaBytes, &full_bar[s]);
          if (second)
            bulk_load(st + kABytes + kBBytes + 2 * kSfaBytes, sfb0 + (p.sf_k_atoms + (int64_t)kt * 4) * 512, kSfaBytes,
                      &full_bar[s]);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer ---------------------------------
    if (lane == 0) {
      // One flat sequence of stages over all of this CTA's tiles.  The scale factors of a stage
      // are put into tensor memory by warps 6-9 (two column sets, used in turn), so the tensor
      // pipe runs MMAs only.
      const int my_tiles = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const int total = my_tiles * p.k_tiles;
      for (int g = 0; g < total; ++g) {
        const int kt = g % p.k_tiles, it = g / p.k_tiles, s = g % kStages, set = g & 1;
        wait_or_abort(&full_bar[s], (g / kStages) & 1, abort_flag, p.status, 32);
        wait_or_abort(&sf_full[set], (g >> 1) & 1, abort_flag, p.status, 35);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (kt == 0) {                                     // the epilogue drained the last tile
          wait_or_abort(acc_empty, (it & 1) ^ 1, abort_flag, p.status, 34);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t st = ring + (uint32_t)s * kStageBytes;
        const uint64_t da = desc_sw128(st), db = desc_sw128(st + kABytes);
        const uint32_t sfa_t = tmem_base + kSfaCol + (uint32_t)(g & 1) * kSfSet;
        const uint32_t sfb_t = tmem_base + kSfbCol + (uint32_t)(g & 1) * kSfSet;
#pragma unroll
        for (int k = 0; k < 4; ++k)                        // 64 elements = 32 bytes of K per instruction
          umma_fp4(tmem_base + kAccCol, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), p.idesc, sfa_t + 4u * k,
                   sfb_t + 8u * k, kt > 0 || k > 0);
        umma_commit(&empty_bar[s]);
        umma_commit(&sf_empty[set]);
        if (kt == p.k_tiles - 1) umma_commit(acc_full);
      }
    }
  } else if (warp >= 6) {
    // --------------------------- scale factors -> tensor memory ---------------------------
    // Thread = one lane of tensor memory (quarter warp % 4, lane in the quarter).  A 512-byte atom
    // holds, in its 16-byte line l, the scale bytes of rows l, l + 32, l + 64, l + 96 for the four
    // groups of one MMA: exactly the four columns that lane l of EVERY quarter must hold.  Twelve
    // 16-byte loads and 48 columns stored per stage and thread - what tcgen05.cp would do inside
    // the tensor pipe, where each copy costs MMA issue slots.
    const int my_tiles = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total = my_tiles * p.k_tiles;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    for (int g = 0; g < total; ++g) {
      const int s = g % kStages, set = g & 1;
      wait_or_abort(&full_bar[s], (g / kStages) & 1, abort_flag, p.status, 36);
      wait_or_abort(&sf_empty[set], ((g >> 1) & 1) ^ 1, abort_flag, p.status, 37);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint4* atoms = reinterpret_cast<const uint4*>(smem + (size_t)s * kStageBytes + kABytes + kBBytes) + lane;
      uint32_t v[48];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint4 a = atoms[32 * k], b0 = atoms[32 * (4 + k)], b1 = atoms[32 * (8 + k)];
        v[4 * k] = a.x; v[4 * k + 1] = a.y; v[4 * k + 2] = a.z; v[4 * k + 3] = a.w;
        v[16 + 8 * k] = b0.x; v[17 + 8 * k] = b0.y; v[18 + 8 * k] = b0.z; v[19 + 8 * k] = b0.w;
        v[20 + 8 * k] = b1.x; v[21 + 8 * k] = b1.y; v[22 + 8 * k] = b1.z; v[23 + 8 * k] = b1.w;
      }
      const uint32_t col = lane_base + kSfaCol + (uint32_t)set * kSfSet;       // SFA columns, then SFB right behind
      tmem_st16(col, &v[0]);
      tmem_st16(col + 16u, &v[16]);
      tmem_st16(col + 32u, &v[32]);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) gb_mbar_arrive(&sf_full[set]);
    }
  } else if (warp < 4) {
    // ------------------------------- epilogue -----------------------------------
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int mt = tile % p.m_tiles, n0 = (tile / p.m_tiles) * kBN;
      wait_or_abort(acc_full, it & 1, abort_flag, p.status, 33);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t row = (int64_t)mt * kBM + warp * 32 + lane;
      const bool row_ok = row < p.M;
      const float rs = (p.a_scale && row_ok ? p.a_scale[row] : 1.0f) * p.global_scale;
      uint32_t va[32], vb[32];
      const uint32_t tbase = tmem_base + ((uint32_t)(warp * 32) << 16) + kAccCol;
      tmem_ld32(tbase, va);
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 64) {               // two chunks of 32 columns per pass
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tmem_ld32(tbase + (uint32_t)c0 + 32u, vb);         // in flight while the first chunk is stored
        store_chunk(p, va, row, row_ok, rs, n0 + c0);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 64 < kBN) {
          tmem_ld32(tbase + (uint32_t)c0 + 64u, va);
        } else {
          // every column of the accumulator is in registers: hand it back before the last stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) gb_mbar_arrive(acc_empty);
        }
        store_chunk(p, vb, row, row_ok, rs, n0 + c0 + 32);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// ---- NVFP4 quantisation of activation rows ---------------------------------------------
// The arithmetic of gridbook/codec.py:377-425 with a scale of its own per row, as the
// reference's row quantiser chooses it (gridbook/csrc/cb_fused_fp4_gemm.cu:345-355):
//   gs = (range * 6) / rowmax,  a_scale = 1 / gs,  xs = x * gs,
//   SF = E4M3(min(max|xs| / 6, 448)) per group of sixteen, one rounding,
//   code = E2M1 nearest of clamp(xs / SF, +-6), a tie going to the even code index,
//   sign bit = sign of xs (kept on zeros); a zero SF zeroes its group.
// Every operation is a correctly rounded fp32 one (no approximate reciprocal), so the bytes are
// those of the torch formulation.
// Two fp32 -> one byte of two E2M1 codes (lo in the low nibble): round to nearest, a tie to the
// even code, clamped to +-6, the sign kept on a zero.
GB_DEVINL uint32_t e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{ .reg .b8 t;\n  cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n  cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__global__ void __launch_bounds__(256)
nvfp4_quantize_rows_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sfa,
                           float* __restrict__ a_scale, int64_t M, int64_t K, float range) {
  const int64_t row = blockIdx.x;
  const int64_t groups = K / 16, k_atoms = (groups + 3) / 4;
  auto sf_offset = [&](int64_t g) {
    return (row % 32) * 16 + ((row / 32) % 4) * 4 + (g % 4) + (g / 4) * 512 + (row / 128) * (512 * k_atoms);
  };
  if (row >= M) {                                        // padding rows of the last 128-row tile: zero scales
    for (int64_t g = threadIdx.x; g < groups; g += blockDim.x) sfa[sf_offset(g)] = 0;
    return;
  }
  const uint16_t* xr = x + row * K;
  __shared__ float red[8];
  float amax = 0.0f;
  for (int64_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      amax = fmaxf(amax, fmaxf(fabsf(gb_bf16_bits_to_f32(w[j] & 0xffffu)), fabsf(gb_bf16_bits_to_f32(w[j] >> 16))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const bool live = amax > 0.0f && isfinite(amax);
  const float gs = live ? __fdiv_rn(__fmul_rn(range, 6.0f), amax) : 1.0f;
  if (threadIdx.x == 0) a_scale[row] = live ? __fdiv_rn(1.0f, gs) : 0.0f;
  for (int64_t g = threadIdx.x; g < groups; g += blockDim.x) {
    const uint4 v0 = reinterpret_cast<const uint4*>(xr)[2 * g], v1 = reinterpret_cast<const uint4*>(xr)[2 * g + 1];
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float xs[16];
    float gmax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xs[2 * j] = __fmul_rn(gb_bf16_bits_to_f32(w[j] & 0xffffu), gs);
      xs[2 * j + 1] = __fmul_rn(gb_bf16_bits_to_f32(w[j] >> 16), gs);
      gmax = fmaxf(gmax, fmaxf(fabsf(xs[2 * j]), fabsf(xs[2 * j + 1])));
    }
    const float sf = live ? fminf(__fdiv_rn(gmax, 6.0f), 448.0f) : 0.0f;
    const uint32_t sf_byte = gb_f32_to_e4m3(sf);
    const float sf_f = gb_e4m3_to_f32(sf_byte);
    sfa[sf_offset(g)] = (uint8_t)sf_byte;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t byte;
      if (sf_f != 0.0f) byte = e2m1x2(__fdiv_rn(xs[2 * j], sf_f), __fdiv_rn(xs[2 * j + 1], sf_f));
      else byte = ((__float_as_uint(xs[2 * j]) >> 31) << 3) | ((__float_as_uint(xs[2 * j + 1]) >> 31) << 7);
      if (j < 4) lo |= byte << (8 * j);
      else hi |= byte << (8 * (j - 4));
    }
    reinterpret_cast<uint2*>(packed + row * (K / 2))[g] = make_uint2(lo, hi);
  }
}

}  // namespace

int gb_prepare_gemm_fp4() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemm_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  return GB_OK;
}

extern "C" {

int64_t gb_nvfp4_sf_bytes(int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0) return 0;
  return ((rows + 127) / 128) * ((K / 16 + 3) / 4) * 512;
}

int gb_nvfp4_quantize_rows(const void* x, int64_t M, int64_t K, float range, void* packed, void* sf, float* a_scale,
                           void* stream) {
  GB_REQUIRE(x && packed && sf && a_scale, "null pointer argument");
  GB_REQUIRE(M >= 0 && K > 0 && K % 16 == 0, "bad shape M=%lld K=%lld (K a multiple of 16)", (long long)M, (long long)K);
  GB_REQUIRE(((uintptr_t)x & 15u) == 0 && ((uintptr_t)packed & 7u) == 0, "rows must be 16-byte aligned");
  GB_REQUIRE(range > 0.0f && range <= 448.0f, "range multiplier %g outside (0, 448]", (double)range);
  if (M == 0) return GB_OK;
  const int64_t padded = (M + 127) / 128 * 128;
  gb_count_launch();
  nvfp4_quantize_rows_kernel<<<(unsigned)padded, 256, 0, (cudaStream_t)stream>>>(
      (const uint16_t*)x, (uint8_t*)packed, (uint8_t*)sf, a_scale, M, K, range);
  GB_LAUNCH_OK("nvfp4_quantize_rows_kernel");
  return GB_OK;
}

int gb_gemm_fp4(const void* A, const void* sfa, const void* B, const void* sfb, void* D, int64_t M, int64_t N, int64_t K,
                const float* a_scale, float global_scale, void* stream) {
  GB_REQUIRE(A && sfa && B && sfb && D, "null pointer argument");
  GB_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 256 == 0, "K=%lld must be a multiple of 256", (long long)K);
  GB_REQUIRE(((uintptr_t)A & 15u) == 0 && ((uintptr_t)B & 15u) == 0 && ((uintptr_t)D & 15u) == 0 &&
             ((uintptr_t)sfa & 15u) == 0 && ((uintptr_t)sfb & 15u) == 0, "operands must be 16-byte aligned");
  GB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "dimension too large");
  if (M == 0) return GB_OK;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  CUtensorMap map_a, map_b;
  int rc = gb_tensor_map_operand(&map_a, A, M, K / 2, 1, kBM);
  if (rc != GB_OK) return rc;
  rc = gb_tensor_map_operand(&map_b, B, N, K / 2, 1, kBN);
  if (rc != GB_OK) return rc;
  Fp4Params p = {};
  p.M = M; p.N = N; p.K = K;
  p.k_tiles = (int)(K / 256);
  p.m_tiles = (int)((M + kBM - 1) / kBM);
  p.n_tiles = (int)((N + kBN - 1) / kBN);
  p.sf_k_atoms = K / 64;
  p.sfa = (const uint8_t*)sfa;
  p.sfb = (const uint8_t*)sfb;
  p.a_scale = a_scale;
  p.global_scale = global_scale == 0.0f ? 1.0f : global_scale;
  // block-scaled instruction descriptor: E2M1 x E2M1, both K-major, UE4M3 scale factors, N >> 3, M >> 4
  p.idesc = (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.D = (uint16_t*)D;
  p.status = gb_status_word();
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  GB_REQUIRE(tiles < (1ll << 31), "too many output tiles");
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  gb_count_launch();
  gemm_fp4_kernel<<<grid, kThreads, kSmem, (cudaStream_t)stream>>>(map_a, map_b, p);
  GB_LAUNCH_OK("gemm_fp4_kernel");
  return GB_OK;
}

}  // extern "C"
