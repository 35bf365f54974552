// Prefill GEMM on the 5th-generation tensor cores: D[M,N] = A[M,K] . B[N,K]^T with both
// operands K-major, bf16 x bf16 (kind::f16) or E4M3 x E4M3 (kind::f8f6f4), fp32 accumulators
// in tensor memory, scaled bf16 epilogue.
//
// Persistent CTAs (one per SM) walk the 128 x 256 output tiles, M fastest.  Warp 4 (one
// thread) streams 128-byte-wide K slabs of A and B into a shared-memory ring with tiled TMA
// loads (128-byte swizzle); warp 5 (one thread) issues tcgen05.mma on shared-memory matrix
// descriptors and releases ring stages with tcgen05.commit; warps 0..3 read the accumulator
// out of tensor memory (tcgen05.ld, one 32-lane quarter each), apply the row / column /
// global scales and store bf16.  Tensor memory holds TWO accumulators (512 columns): while
// the epilogue warps drain one, the MMAs of the next tile already fill the other, and the
// TMA ring never drains between tiles.  B is the decoded weight tile the expanders write (gb_expand_fp8 /
// gb_expand_fp4_bf16); A is the bucketed activation matrix.
//
// Grouped mode (routed prefill): A holds the routed rows sorted by expert, B the decoded stack
// [E*N, K]; expert e owns rows [seg[e], seg[e+1]) of A.  Every CTA builds the per-expert tile
// prefix from the device-side segment offsets (no host read), walks tiles N fastest so the CTAs
// running together share an expert's decoded weights through L2, and the epilogue masks the
// rows past the segment end (a row tile may run into the next expert's rows) and can scatter
// its rows through a row map.
#include "gb_common.cuh"

#include <cuda.h>
#include <mutex>

namespace {

constexpr int kBM = 128, kBN = 256;
constexpr int kSlabBytes = 128;                    // K bytes per row per stage (one swizzle span)
constexpr int kStageBytes = (kBM + kBN) * kSlabBytes;   // 48 KiB
constexpr int kStages = 4;
constexpr int kTmemCols = 512;                     // two 128 x 256 fp32 accumulators
constexpr int kGemmThreads = 192;
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /* alignment */ + 256 /* barriers */;
constexpr int kMaxGroups = 1024;                   // experts of one grouped launch
constexpr int kGroupSmem = 2 * (kMaxGroups + 1) * 4 + 8;   // segment offsets + row-tile prefix

struct GemmParams {
  int64_t M, N, K;
  int k_tiles;
  int m_tiles, n_tiles;      // output tiles along M and N
  int elem_bytes;            // 2 (bf16) or 1 (e4m3)
  uint32_t idesc;
  const float* a_scale;      // [M] or null
  const float* b_scale;      // [N] or null
  float global_scale;
  uint16_t* D;
  int* status;
  // grouped mode
  const int32_t* seg;        // [E+1] first sorted row of every expert, seg[E] = routed rows
  const int32_t* row_map;    // [P] output row of a sorted row, or null = identity
  int E;
};

// One output tile of either mode: first A row, end of the valid rows, first B row, first
// output column, and the B-scale offset of the expert.
struct Tile {
  int m0, m_end, b_row0, n0, scale0;
};

template <bool kGrouped>
GB_DEVINL Tile tile_of(const GemmParams& p, int tile, const int* seg_s, const int* base_s) {
  Tile t;
  if (!kGrouped) {
    t.m0 = (tile % p.m_tiles) * kBM;
    t.n0 = (tile / p.m_tiles) * kBN;
    t.m_end = (int)p.M;
    t.b_row0 = t.n0;
    t.scale0 = 0;
  } else {
    const int gm = tile / p.n_tiles;
    t.n0 = (tile % p.n_tiles) * kBN;
    int lo = 0, hi = p.E;                 // largest e with base_s[e] <= gm
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (base_s[mid] <= gm) lo = mid; else hi = mid;
    }
    t.m0 = seg_s[lo] + (gm - base_s[lo]) * kBM;
    t.m_end = seg_s[lo + 1];
    t.scale0 = lo * (int)p.N;
    t.b_row0 = t.scale0 + t.n0;
  }
  return t;
}

GB_DEVINL void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(gb_smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(gb_smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart.
GB_DEVINL uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
  d |= (uint64_t)(1024u >> 4) << 32;                      // stride between 8-row groups
  d |= (uint64_t)1 << 46;                                 // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                                 // 128-byte swizzle
  return d;
}

GB_DEVINL void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate, bool fp8) {
  if (fp8) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
  }
}

GB_DEVINL void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(gb_smem_u32(bar)) : "memory");
}

// A bounded wait that remembers a timeout for the rest of the CTA: later waits return at once.
GB_DEVINL void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (*abort_flag) return;
  if (!gb_mbar_wait(bar, parity)) {
    *abort_flag = 1;
    atomicExch(status, code);
  }
}

template <bool kGrouped>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;                                                   // kStages x (A slab | B slab)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;          // [2] accumulator complete (one commit)
  uint64_t* acc_empty = acc_full + 2;                // [2] accumulator drained (four epilogue warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* seg_s = reinterpret_cast<int*>(smem + kStages * kStageBytes + 256);   // [E+1], grouped mode
  int* base_s = seg_s + kMaxGroups + 1;                                       // [E+1] row-tile prefix

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool fp8 = p.elem_bytes == 1;
  if (kGrouped && warp == 0) {
    // row tiles of expert e: ceil(rows / 128); exclusive prefix by one warp, 32 experts a pass
    int carry = 0;
    for (int e0 = 0; e0 < p.E; e0 += 32) {
      const int e = e0 + lane;
      const int lo = e < p.E ? p.seg[e] : 0, hi = e < p.E ? p.seg[e + 1] : 0;
      int tiles = (hi - lo + kBM - 1) / kBM, incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (e < p.E) {
        seg_s[e] = lo;
        base_s[e] = carry + incl - tiles;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      seg_s[p.E] = p.seg[p.E];
      base_s[p.E] = carry;
    }
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      gb_mbar_init(&full_bar[s], 1);
      gb_mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      gb_mbar_init(&acc_full[b], 1);
      gb_mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0;
    gb_fence_barrier_init();
  }
  if (warp == 5) {   // tensor memory for two 128 x 256 fp32 accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(gb_smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = kGrouped ? base_s[p.E] * p.n_tiles : p.m_tiles * p.n_tiles;

  // Every role walks the same tile sequence: tile = blockIdx.x, + gridDim.x, ...; M tiles vary
  // fastest, so the CTAs working at the same time share a few B (weight) tiles and sweep A,
  // which fits L2: the decoded weight tile is read from HBM once.
  if (warp == 4) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      const int slab_elems = kSlabBytes / p.elem_bytes;
      int kk = 0;                                        // K slabs issued so far, over all tiles
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const Tile t = tile_of<kGrouped>(p, tile, seg_s, base_s);
        for (int kt = 0; kt < p.k_tiles; ++kt, ++kk) {
          const int s = kk % kStages;
          wait_or_abort(&empty_bar[s], ((kk / kStages) & 1) ^ 1, abort_flag, p.status, 11);
          gb_mbar_expect_tx(&full_bar[s], kStageBytes);
          uint8_t* a_dst = ring + (size_t)s * kStageBytes;
          tma_load_2d(a_dst, &map_a, kt * slab_elems, t.m0, &full_bar[s]);
          tma_load_2d(a_dst + kBM * kSlabBytes, &map_b, kt * slab_elems, t.b_row0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------- MMA issuer ---------------------------------
    if (lane == 0) {
      int kk = 0, it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        // the epilogue must have drained this accumulator (its use two tiles ago)
        wait_or_abort(&acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, p.status, 14);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kBN);
        for (int kt = 0; kt < p.k_tiles; ++kt, ++kk) {
          const int s = kk % kStages;
          wait_or_abort(&full_bar[s], (kk / kStages) & 1, abort_flag, p.status, 12);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = gb_smem_u32(ring + (size_t)s * kStageBytes);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + kBM * kSlabBytes);
#pragma unroll
          for (int k = 0; k < kSlabBytes / 32; ++k)       // 32 bytes of K per instruction
            umma(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), p.idesc, kt > 0 || k > 0, fp8);
          umma_commit(&empty_bar[s]);                      // stage free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);                       // accumulator complete
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const Tile t = tile_of<kGrouped>(p, tile, seg_s, base_s);
      const int n0 = t.n0;
      wait_or_abort(&acc_full[buf], (it >> 1) & 1, abort_flag, p.status, 13);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t row = (int64_t)t.m0 + warp * 32 + lane;
      const bool row_ok = row < t.m_end;
      const float rs = (p.a_scale && row_ok ? p.a_scale[row] : 1.0f) * p.global_scale;
      const float* b_scale = p.b_scale ? p.b_scale + t.scale0 : nullptr;
      const int64_t out_row = kGrouped && p.row_map && row_ok ? p.row_map[row] : row;
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(buf * kBN + c0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 == kBN) {
          // every column of this accumulator is in registers: hand it back before the stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) gb_mbar_arrive(&acc_empty[buf]);
        }
        if (row_ok) {
          uint16_t* out = p.D + out_row * p.N + n0 + c0;
          const int64_t ncol = p.N - (n0 + c0);
          if (ncol >= 32 && (p.N % 8) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int c = q * 8 + j * 2;
                const float s0 = b_scale ? b_scale[n0 + c0 + c] : 1.0f;
                const float s1 = b_scale ? b_scale[n0 + c0 + c + 1] : 1.0f;
                w[j] = gb_f32_to_bf16_bits(__uint_as_float(v[c]) * rs * s0) |
                       (gb_f32_to_bf16_bits(__uint_as_float(v[c + 1]) * rs * s1) << 16);
              }
              *reinterpret_cast<uint4*>(out + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
            for (int c = 0; c < 32 && c < ncol; ++c) {
              const float s0 = b_scale ? b_scale[n0 + c0 + c] : 1.0f;
              out[c] = (uint16_t)gb_f32_to_bf16_bits(__uint_as_float(v[c]) * rs * s0);
            }
          }
        }
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

// ---- per-token E4M3 quantisation of the activations (fp8-grid prefill) ----------------
__global__ void __launch_bounds__(256)
fp8_quantize_rows_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale_out,
                         int64_t K, int scale_rule) {
  const uint16_t* row = x + (int64_t)blockIdx.x * K;
  uint8_t* qrow = q + (int64_t)blockIdx.x * K;
  __shared__ float red[8];
  __shared__ float s_scale;
  float amax = 0.0f;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(gb_bf16_bits_to_f32(row[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int w = 1; w < 8; ++w) a = fmaxf(a, red[w]);
    const float s = scale_rule == GB_SCALE_RULE_DIV ? __fdiv_rn(a, 448.0f) : __fmul_rn(a, 1.0f / 448.0f);
    s_scale = fmaxf(s, 1.0f / (448.0f * 512.0f));
    scale_out[blockIdx.x] = s_scale;
  }
  __syncthreads();
  const float scale = s_scale;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
    const float v = gb_bf16_bits_to_f32(row[i]);
    qrow[i] = (uint8_t)gb_f32_to_e4m3(fminf(fmaxf(__fdiv_rn(v, scale), -448.0f), 448.0f));
  }
}

// ---- routed prefill helpers: rows in expert order ---------------------------------------
// out[j] = x[x_row[order[j]]] (or x[order[j]] without x_row) for the sorted rows j < *n_rows.
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ x_row,
                       const int32_t* __restrict__ order, const int32_t* __restrict__ n_rows, int vecs,
                       uint4* __restrict__ out) {
  const int j = blockIdx.x;
  if (j >= *n_rows) return;
  const int pair = order[j];
  const int64_t src = x_row ? x_row[pair] : pair;
  const uint4* in = x + src * vecs;
  uint4* o = out + (int64_t)j * vecs;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) o[i] = in[i];
}

// out[j][c] = bf16(bf16(silu(gate)) * up), gate = h[j][c], up = h[j][inter + c]: every torch bf16
// op of the reference chain rounds (F.silu on bf16, then a bf16 multiply).  With kBucket the fp4
// group-16 activation bucket of the next projection is applied to the result in registers (a
// thread holds eight values, its neighbour lane the other half of the group).
template <bool kBucket>
__global__ void __launch_bounds__(128)
moe_swiglu_rows_kernel(const uint4* __restrict__ h, const int32_t* __restrict__ n_rows, int vecs, int scale_rule,
                       uint4* __restrict__ out) {
  const int j = blockIdx.x;
  if (j >= *n_rows) return;
  const uint4* row = h + (int64_t)j * 2 * vecs;
  for (int i0 = 0; i0 < vecs; i0 += blockDim.x) {          // warp-uniform trip count: the bucket shuffles
    const int i = i0 + threadIdx.x;
    const bool live = i < vecs;
    const int ii = live ? i : 0;
    const uint4 g = row[ii], u = row[vecs + ii];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t r[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t packed = 0;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const float gate = gb_bf16_bits_to_f32((gw[q] >> (16 * hlf)) & 0xffffu);
        const float up = gb_bf16_bits_to_f32((uw[q] >> (16 * hlf)) & 0xffffu);
        const float sl = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(gate / (1.0f + __expf(-gate))));
        packed |= gb_f32_to_bf16_bits(sl * up) << (16 * hlf);
      }
      r[q] = packed;
    }
    uint4 res = make_uint4(r[0], r[1], r[2], r[3]);
    if (kBucket) res = gb_fp4_group16_qdq_pair(res, scale_rule);
    if (live) out[(int64_t)j * vecs + i] = res;
  }
}

// ---- tensor maps ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::mutex g_encode_mutex;
EncodeTiledFn g_encode = nullptr;

int get_encoder(EncodeTiledFn* out) {
  std::lock_guard<std::mutex> lock(g_encode_mutex);
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    GB_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess)
      return gb_fail(GB_ECUDA, "the driver does not export cuTensorMapEncodeTiled");
    g_encode = (EncodeTiledFn)fn;
  }
  *out = g_encode;
  return GB_OK;
}

int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int elem_bytes, int box_rows) {
  EncodeTiledFn enc;
  int rc = get_encoder(&enc);
  if (rc != GB_OK) return rc;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(kSlabBytes / elem_bytes), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gb_fail(GB_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return GB_OK;
}

}  // namespace

// Plain (unswizzled) byte tensor map over [rows][pitch_bytes], for kernels that stream
// row slices of a packed weight matrix.  `map_out` points at a CUtensorMap.
int gb_tensor_map_bytes_2d(void* map_out, const void* base, uint64_t inner_bytes, uint64_t rows,
                           uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows) {
  EncodeTiledFn enc;
  int rc = get_encoder(&enc);
  if (rc != GB_OK) return rc;
  const cuuint64_t dims[2] = {(cuuint64_t)inner_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return gb_fail(GB_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return GB_OK;
}

int gb_tensor_map_operand(void* map_out, const void* base, int64_t rows, int64_t K, int elem_bytes, int box_rows) {
  return make_map((CUtensorMap*)map_out, base, rows, K, elem_bytes, box_rows);
}

int gb_prepare_gemm() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemm_tn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kGemmSmem));
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemm_tn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kGemmSmem + kGroupSmem));
  return GB_OK;
}

extern "C" {

int gb_fp8_quantize_rows(const void* x, void* q, float* scale, int64_t M, int64_t K, int scale_rule, void* stream) {
  GB_REQUIRE(x && q && scale, "null pointer argument");
  GB_REQUIRE(M >= 0 && K > 0, "bad shape M=%lld K=%lld", (long long)M, (long long)K);
  if (M == 0) return GB_OK;
  gb_count_launch();
  fp8_quantize_rows_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, (uint8_t*)q, scale, K,
                                                                        scale_rule);
  GB_LAUNCH_OK("fp8_quantize_rows_kernel");
  return GB_OK;
}

int gb_gemm_tn(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K, int kind, const float* a_scale,
               const float* b_scale, float global_scale, void* stream) {
  GB_REQUIRE(A && B && D, "null pointer argument");
  GB_REQUIRE(kind == GB_GEMM_BF16 || kind == GB_GEMM_E4M3, "unknown gemm kind %d", kind);
  const int eb = kind == GB_GEMM_BF16 ? 2 : 1;
  GB_REQUIRE(M > 0 && N > 0 && K > 0 && (K * eb) % kSlabBytes == 0, "K=%lld must be a multiple of %d elements",
             (long long)K, kSlabBytes / eb);
  GB_REQUIRE(((uintptr_t)A & 15u) == 0 && ((uintptr_t)B & 15u) == 0 && ((uintptr_t)D & 15u) == 0,
             "operands must be 16-byte aligned");
  GB_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "dimension too large");
  if (gb_sm_count() <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, A, M, K, eb, kBM);
  if (rc != GB_OK) return rc;
  rc = make_map(&map_b, B, N, K, eb, kBN);
  if (rc != GB_OK) return rc;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.k_tiles = (int)(K * eb / kSlabBytes);
  p.m_tiles = (int)((M + kBM - 1) / kBM);
  p.n_tiles = (int)((N + kBN - 1) / kBN);
  p.elem_bytes = eb;
  // instruction descriptor: fp32 accumulate, A/B format, both K-major, N >> 3, M >> 4
  p.idesc = (1u << 4) | ((kind == GB_GEMM_BF16 ? 1u : 0u) << 7) | ((kind == GB_GEMM_BF16 ? 1u : 0u) << 10) |
            ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.global_scale = global_scale == 0.0f ? 1.0f : global_scale;
  p.D = (uint16_t*)D;
  p.status = gb_status_word();
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  GB_REQUIRE(tiles < (1ll << 31), "too many output tiles");
  const int sms = gb_sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));          // persistent: one CTA per SM
  gb_count_launch();
  gemm_tn_kernel<false><<<grid, kGemmThreads, kGemmSmem, (cudaStream_t)stream>>>(map_a, map_b, p);
  GB_LAUNCH_OK("gemm_tn_kernel");
  return GB_OK;
}

int gb_gemm_tn_grouped(const void* A, const void* B, void* D, int64_t P, int64_t N, int64_t K, int kind, int64_t E,
                       const int32_t* seg_offsets, const int32_t* row_map, const float* a_scale, const float* b_scale,
                       float global_scale, void* stream) {
  GB_REQUIRE(A && B && D && seg_offsets, "null pointer argument");
  GB_REQUIRE(kind == GB_GEMM_BF16 || kind == GB_GEMM_E4M3, "unknown gemm kind %d", kind);
  const int eb = kind == GB_GEMM_BF16 ? 2 : 1;
  GB_REQUIRE(P >= 0 && N > 0 && K > 0 && (K * eb) % kSlabBytes == 0, "K=%lld must be a multiple of %d elements",
             (long long)K, kSlabBytes / eb);
  GB_REQUIRE(E > 0 && E <= kMaxGroups, "expert count %lld outside [1, %d]", (long long)E, kMaxGroups);
  GB_REQUIRE(((uintptr_t)A & 15u) == 0 && ((uintptr_t)B & 15u) == 0 && ((uintptr_t)D & 15u) == 0,
             "operands must be 16-byte aligned");
  GB_REQUIRE(P < (1ll << 30) && E * N < (1ll << 31) && K < (1ll << 31), "dimension too large");
  if (P == 0) return GB_OK;
  if (gb_sm_count() <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  CUtensorMap map_a, map_b;
  int rc = make_map(&map_a, A, P, K, eb, kBM);
  if (rc != GB_OK) return rc;
  rc = make_map(&map_b, B, E * N, K, eb, kBN);
  if (rc != GB_OK) return rc;
  GemmParams p = {};
  p.M = P; p.N = N; p.K = K;
  p.k_tiles = (int)(K * eb / kSlabBytes);
  p.m_tiles = 0;                                   // counted on the device from seg_offsets
  p.n_tiles = (int)((N + kBN - 1) / kBN);
  p.elem_bytes = eb;
  p.idesc = (1u << 4) | ((kind == GB_GEMM_BF16 ? 1u : 0u) << 7) | ((kind == GB_GEMM_BF16 ? 1u : 0u) << 10) |
            ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.global_scale = global_scale == 0.0f ? 1.0f : global_scale;
  p.D = (uint16_t*)D;
  p.status = gb_status_word();
  p.seg = seg_offsets; p.row_map = row_map; p.E = (int)E;
  // at most ceil(P/128) + E row tiles, whatever the routing
  const int64_t tiles = ((P + kBM - 1) / kBM + E) * p.n_tiles;
  GB_REQUIRE(tiles < (1ll << 31), "too many output tiles");
  const int sms = gb_sm_count();
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  gb_count_launch();
  gemm_tn_kernel<true><<<grid, kGemmThreads, kGemmSmem + kGroupSmem, (cudaStream_t)stream>>>(map_a, map_b, p);
  GB_LAUNCH_OK("gemm_tn_kernel<grouped>");
  return GB_OK;
}

int gb_moe_gather_rows(const void* x, const int32_t* x_row, const int32_t* order, const int32_t* seg_offsets,
                       int64_t E, int64_t P, int64_t K, void* out, void* stream) {
  GB_REQUIRE(x && order && seg_offsets && out, "null pointer argument");
  GB_REQUIRE(P >= 0 && E > 0 && K > 0 && K % 8 == 0, "bad shape P=%lld E=%lld K=%lld", (long long)P, (long long)E,
             (long long)K);
  GB_REQUIRE(((uintptr_t)x & 15u) == 0 && ((uintptr_t)out & 15u) == 0, "rows must be 16-byte aligned");
  if (P == 0) return GB_OK;
  gb_count_launch();
  moe_gather_rows_kernel<<<(unsigned)P, 128, 0, (cudaStream_t)stream>>>(
      (const uint4*)x, x_row, order, seg_offsets + E, (int)(K / 8), (uint4*)out);
  GB_LAUNCH_OK("moe_gather_rows_kernel");
  return GB_OK;
}

int gb_moe_swiglu_rows(const void* h, const int32_t* seg_offsets, int64_t E, int64_t P, int64_t inter, int act,
                       int scale_rule, void* out, void* stream) {
  GB_REQUIRE(h && seg_offsets && out, "null pointer argument");
  GB_REQUIRE(P >= 0 && E > 0 && inter > 0 && inter % 8 == 0, "bad shape P=%lld E=%lld inter=%lld", (long long)P,
             (long long)E, (long long)inter);
  GB_REQUIRE(act == GB_ACT_NONE || (act == GB_ACT_FP4_GROUP16 && inter % 16 == 0),
             "the fused bucket is the fp4 group-16 one and wants inter %% 16 == 0");
  GB_REQUIRE(((uintptr_t)h & 15u) == 0 && ((uintptr_t)out & 15u) == 0, "rows must be 16-byte aligned");
  if (P == 0) return GB_OK;
  gb_count_launch();
  const int vecs = (int)(inter / 8);
  const unsigned threads = vecs >= 128 ? 128u : (unsigned)((vecs + 31) / 32 * 32);   // whole warps, few idle lanes
  if (act == GB_ACT_FP4_GROUP16)
    moe_swiglu_rows_kernel<true><<<(unsigned)P, threads, 0, (cudaStream_t)stream>>>(
        (const uint4*)h, seg_offsets + E, (int)(inter / 8), scale_rule, (uint4*)out);
  else
    moe_swiglu_rows_kernel<false><<<(unsigned)P, threads, 0, (cudaStream_t)stream>>>(
        (const uint4*)h, seg_offsets + E, (int)(inter / 8), scale_rule, (uint4*)out);
  GB_LAUNCH_OK("moe_swiglu_rows_kernel");
  return GB_OK;
}

}  // extern "C"
