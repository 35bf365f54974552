// M = 1 linear for the literal format (fp4 grid, full mode, k = 8, E4M3-direct scales) by
// inner-product tables.
//
// With one 256-entry codebook and one activation row, a codeword's contribution to the dot
// product can only take 256 values per position: T[s][c][v] = <codebook[c], x[256 s + 8 v ..+8]>.
// A CTA owns four superblock columns of K and a band of rows.  It builds T for its columns
// once (tensor cores: activation segments x codebook, 128 KiB of fp32 in shared memory; the
// fp4 activation bucket is applied on the way in), then streams its rows' 192-byte slices
// through a TMA ring.  Per superblock a lane owns four codewords (two groups): one 32-bit load
// of codes, four table lookups, one 16-bit load of scales, two adds and two scaled
// accumulates - nine instructions per 16 weights against ~270 for expanding every weight,
// which is what lets a 1.5-bit format approach the HBM stream.
//
// Shared-memory geometry.  A table row is 256 bytes: one codeword, two superblock columns, 32
// positions each; columns {0,1} fill one 64 KiB region, columns {2,3} the next, and the
// regions start on 64 KiB boundaries of the shared window.  A lookup address is then the
// lane's constant (region + position) with the code dropped into byte 1: one byte permute,
// no shift, no add.  The bank of a lookup is its position alone.  Eight lanes walk one row,
// so a warp takes four rows at a time; row r of the four reads its positions in the order
// j = q ^ r (q = 0..3), and rows 2,3 work two superblock columns ahead of rows 0,1, which
// makes the code loads, the scale loads and all four lookups of a warp conflict-free.
//
// K slices write their partial sums to their own slot; a second tiny kernel adds the slots,
// applies the global scale and rounds to bf16 once.
#include "gb_common.cuh"

#include <cuda.h>


namespace {

constexpr int kS = 4;                         // superblock columns per CTA
constexpr int kConsumers = 16;                // warps (24 also fits the layout; measured no faster)
constexpr int kBlocksPerWarp = 2;             // eight-code blocks of the table a warp builds per column: w, w + kConsumers
constexpr int kDotThreads = (kConsumers + 1) * 32;
constexpr int kStageRows = 4 * kConsumers;    // 64 rows per stage, four per warp
constexpr int kRowBytes = kS * 48;            // 192 bytes of each row per stage
constexpr int kStageBytes = kStageRows * kRowBytes;
constexpr int kDotStages = 6 * 16 / kConsumers;
static_assert(kConsumers == 16 || kConsumers == 24, "stage geometry is laid out for 16 or 24 consumer warps");
constexpr int kFrontStages = kDotStages - 1;  // ring stages in front of the tables, the rest behind
constexpr uint32_t kRegion = 0x10000u;        // 64 KiB: 256 codes x 256-byte rows
constexpr int kTableBytes = 2 * (int)kRegion;
constexpr int kBackBytes = (kDotStages - kFrontStages) * kStageBytes + kS * 512 + 256;
// Front ring + alignment slack up to the first 64 KiB boundary, tables, back part.  The
// kernel checks at run time that the window it was given really holds this layout.
constexpr int kDotSmem = (int)kRegion + kTableBytes + kBackBytes;
static_assert(kFrontStages * kStageBytes + 4096 <= (int)kRegion, "front ring must end before the first boundary");

struct DotParams {
  const uint16_t* x;        // [K] bf16
  const uint16_t* codebook; // [256 * 8] bf16
  int act, scale_rule;
  int64_t N;
  int n_sb, n_slices, n_groups, rows_per_group;
  float* ws;                // [n_slices][N] partial sums; pair mode: [n_slices][P][N]
  int* status;
  // ---- pair mode: one independent GEMV per routed (token, expert) pair ----
  const int32_t* pair_expert;   // [P] global expert id of every pair (outside [base, base+E): skipped)
  const int32_t* x_row;         // [P] activation row of every pair (nullptr: the pair index)
  int P, E, expert_base, bands; // bands: row bands per pair
  uint16_t* y;                  // direct bf16 output when there is one K slice and no SwiGLU
  uint16_t* y_peer[8];          // optional: pair p's row lives in y_peer[p / pairs_per_rank]
  int pairs_per_rank;
  int direct;                   // 1: store y from the kernel, 0: partial sums + the summing kernel
  float global_scale;
  // pair mode, second projection of an MLP: the activation row of pair p is
  // silu(gate) * up of the FIRST projection's partial sums (its K slices still unsummed)
  const float* xws;             // [xws_slices][P][xws_N] partial sums of the gate/up projection, or nullptr
  int xws_slices;
  int64_t xws_N;                // rows of the gate/up projection (= 2 x this projection's K)
  float xws_scale;              // its global scale
};

// Output row of pair `pair` (width `width` elements): in y, or in its home rank's buffer.
GB_DEVINL uint16_t* pair_out_row(const DotParams& p, int pair, int64_t width) {
  if (p.pairs_per_rank > 0) {
    const int home = pair / p.pairs_per_rank;
    return p.y_peer[home] + (int64_t)(pair - home * p.pairs_per_rank) * width;
  }
  return p.y + (int64_t)pair * width;
}

// Shared-memory loads that depend on a token (the result of the barrier wait that made the
// data visible): plain asm the scheduler may reorder freely, but never above that wait.
template <int kImm>
GB_DEVINL float ldt_f32(uint32_t a, uint32_t tok) {
  float v;
  asm("ld.shared.f32 %0, [%1+%2]; // %3" : "=f"(v) : "r"(a), "n"(kImm), "r"(tok));
  return v;
}
template <int kImm>
GB_DEVINL uint32_t ldt_u32(uint32_t a, uint32_t tok) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2]; // %3" : "=r"(v) : "r"(a), "n"(kImm), "r"(tok));
  return v;
}
template <int kImm>
GB_DEVINL uint32_t ldt_u16(uint32_t a, uint32_t tok) {
  uint32_t v;
  asm("{ .reg .u16 t; ld.shared.u16 t, [%1+%2]; cvt.u32.u16 %0, t; } // %3" : "=r"(v) : "r"(a), "n"(kImm), "r"(tok));
  return v;
}
// Two E4M3 bytes (low 16 bits of w) -> two fp32, exactly (subnormal codes included).
GB_DEVINL void e4m3x2_to_f32(uint32_t w, float& lo, float& hi) {
  asm("{ .reg .b16 p, l, h; .reg .b32 q;\n"
      "  cvt.u16.u32 p, %2;\n"
      "  cvt.rn.f16x2.e4m3x2 q, p;\n"
      "  mov.b32 {l, h}, q;\n"
      "  cvt.f32.f16 %0, l;\n"
      "  cvt.f32.f16 %1, h; }"
      : "=f"(lo), "=f"(hi) : "r"(w));
}

// One superblock column of one row for this lane's two groups.  `rowp` already points at the
// lane's superblock; kOff is the column's offset inside a table row (0 or 128).
template <int kPtrOff, int kTabOff>
GB_DEVINL void dot_superblock(uint32_t rowp_codes, uint32_t rowp_scales, const uint32_t (&base)[4], const uint32_t (&sel)[4],
                              uint32_t sel_sc, uint32_t tok, float& acc0, float& acc1) {
  const uint32_t codes = ldt_u32<kPtrOff>(rowp_codes, tok);
  const uint32_t sc = ldt_u16<kPtrOff + 32>(rowp_scales, tok);
  const float t0 = ldt_f32<kTabOff>(__byte_perm(codes, base[0], sel[0]), tok);
  const float t1 = ldt_f32<kTabOff>(__byte_perm(codes, base[1], sel[1]), tok);
  const float t2 = ldt_f32<kTabOff>(__byte_perm(codes, base[2], sel[2]), tok);
  const float t3 = ldt_f32<kTabOff>(__byte_perm(codes, base[3], sel[3]), tok);
  float f01, f23;
  e4m3x2_to_f32(__byte_perm(sc, 0u, sel_sc), f01, f23);
  acc0 = fmaf(t0 + t1, f01, acc0);
  acc1 = fmaf(t2 + t3, f23, acc1);
}

template <bool kPairs>
__global__ void __launch_bounds__(kDotThreads, 1)
gemv_dot_kernel(const __grid_constant__ CUtensorMap map_w, const DotParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base_s = gb_smem_u32(smem);
  // absolute shared addresses of the layout
  const uint32_t tab_s = (base_s + kFrontStages * kStageBytes + (kRegion - 1)) & ~(kRegion - 1);
  const uint32_t back_s = tab_s + kTableBytes;
  if (back_s + kBackBytes > base_s + kDotSmem) {       // same verdict in every thread, before any barrier
    if (threadIdx.x == 0) atomicExch(p.status, 23);
    return;
  }
  uint8_t* table_b = smem + (tab_s - base_s);
  uint8_t* back = smem + (back_s - base_s);
  uint16_t* xq = reinterpret_cast<uint16_t*>(back + (kDotStages - kFrontStages) * kStageBytes);    // kS * 256 bf16
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xq) + kS * 512);
  uint64_t* empty_bar = full_bar + kDotStages;
  auto stage_addr = [&](int s) -> uint32_t {
    return s < kFrontStages ? base_s + (uint32_t)s * kStageBytes : back_s + (uint32_t)(s - kFrontStages) * kStageBytes;
  };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x % p.n_slices;
  // dense: a row band of the matrix; pair mode: (pair, row band of that pair's expert)
  const int group = kPairs ? (int)(blockIdx.x / p.n_slices) % p.bands : (int)(blockIdx.x / p.n_slices);
  const int pair = kPairs ? (int)(blockIdx.x / p.n_slices) / p.bands : 0;
  const int sb0 = slice * kS;
  const int ns = min(kS, p.n_sb - sb0);
  const int64_t row_begin = (int64_t)group * p.rows_per_group;
  const int64_t row_end = min(p.N, row_begin + p.rows_per_group);
  const int n_stages = row_end > row_begin ? (int)((row_end - row_begin + kStageRows - 1) / kStageRows) : 0;

  if (tid == 0) {
    for (int s = 0; s < kDotStages; ++s) {
      gb_mbar_init(&full_bar[s], 1);
      gb_mbar_init(&empty_bar[s], kConsumers);
    }
    gb_fence_barrier_init();
  }
  __syncthreads();
  gb_pdl_launch_dependents();

  int64_t tma_row0 = row_begin;          // first row of the band in the tensor map's row space
  const uint16_t* xsrc = p.x;
  if constexpr (kPairs) {
    gb_pdl_wait();                       // the routing and the activations come from earlier kernels
    const int e = p.pair_expert ? p.pair_expert[pair] - p.expert_base : 0;
    if (e < 0 || e >= p.E) return;       // padded route, or an expert another rank holds: whole CTA leaves
    tma_row0 = (int64_t)e * p.N + row_begin;
    xsrc = p.x + (int64_t)(p.x_row ? p.x_row[pair] : pair) * ((int64_t)p.n_sb * 256);
  }

  if (warp == kConsumers) {
    // ------------------------------ producer ------------------------------
    // The weight stream depends on nothing an earlier kernel wrote: the ring fills while the
    // kernel before this one is still finishing.
    if (lane == 0) {
      for (int st = 0; st < n_stages; ++st) {
        const int s = st % kDotStages;
        if (!gb_mbar_wait(&empty_bar[s], ((st / kDotStages) & 1) ^ 1)) {
          gb_pdl_wait();
          atomicExch(p.status, 21);
        }
        gb_mbar_expect_tx(&full_bar[s], kStageBytes);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(stage_addr(s)), "l"(reinterpret_cast<uint64_t>(&map_w)),
              "r"(sb0 * 48), "r"((int)(tma_row0 + (int64_t)st * kStageRows)), "r"(gb_smem_u32(&full_bar[s]))
            : "memory");
      }
    }
    return;
  }

  // ---- inner-product tables ----
  // One unit = one superblock column x eight codes x all 32 positions: two MMAs with the
  // activation segments as the 16 rows (A[m][k] = x[8 (16 h + m) + k]) and the eight
  // codewords as the columns (B[k][n] = codebook[c0 + n][k]).  Warp w owns code blocks w and
  // w + kConsumers (where that exists) for every column, so its B fragments are loaded once,
  // before the wait.
  const int g = lane >> 2, t = lane & 3;
  uint32_t bfrag[kBlocksPerWarp];
  {
    const uint32_t* cb32 = reinterpret_cast<const uint32_t*>(p.codebook);
#pragma unroll
    for (int j = 0; j < kBlocksPerWarp; ++j)
      bfrag[j] = warp + j * kConsumers < 32 ? __ldg(cb32 + ((warp + j * kConsumers) * 8 + g) * 4 + t) : 0u;
  }

  // ---- this slice of the activation row, through its bucket, into shared memory ----
  gb_pdl_wait();                       // the activations (and the partial-sum slots) belong to earlier kernels
  if (tid < ns * 128) {                // two values per thread, a bucket group per eight lanes
    uint32_t w;
    if (kPairs && p.xws) {
      // sum the gate/up projection's K slices, SwiGLU with the bf16 roundings of F.silu(gate) * up
      const int64_t j = (int64_t)sb0 * 256 + 2 * tid, half = p.xws_N / 2;
      float g0 = 0.f, g1 = 0.f, u0 = 0.f, u1 = 0.f;
      for (int sl = 0; sl < p.xws_slices; ++sl) {
        const float* slot = p.xws + ((int64_t)sl * p.P + pair) * p.xws_N;
        const float2 gv = *reinterpret_cast<const float2*>(slot + j);
        const float2 uv = *reinterpret_cast<const float2*>(slot + half + j);
        g0 += gv.x; g1 += gv.y; u0 += uv.x; u1 += uv.y;
      }
      auto act1 = [&](float graw, float uraw) {
        const float gate = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(graw * p.xws_scale));
        const float up = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(uraw * p.xws_scale));
        const float sl = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(gate / (1.0f + __expf(-gate))));
        return gb_f32_to_bf16_bits(sl * up);
      };
      w = act1(g0, u0) | (act1(g1, u1) << 16);
    } else {
      w = reinterpret_cast<const uint32_t*>(xsrc + (int64_t)sb0 * 256)[tid];
    }
    if (p.act == GB_ACT_FP4_GROUP16) w = gb_fp4_group16_qdq_lanes(w, p.scale_rule);
    reinterpret_cast<uint32_t*>(xq)[tid] = w;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

  {
    const uint32_t* xq32 = reinterpret_cast<const uint32_t*>(xq);
#pragma unroll
    for (int s = 0; s < kS; ++s) {
      if (s >= ns) break;
      uint32_t a[2][2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a[h][0] = xq32[s * 128 + (16 * h + g) * 4 + t];
        a[h][1] = xq32[s * 128 + (16 * h + g + 8) * 4 + t];
      }
      // T(s, code, pos) lives at region (s >> 1), row `code`, float (s & 1) * 32 + pos
      float* col = reinterpret_cast<float*>(table_b + (size_t)(s >> 1) * kRegion) + (s & 1) * 32 + g;
#pragma unroll
      for (int j = 0; j < kBlocksPerWarp; ++j) {
        if (warp + j * kConsumers >= 32) break;            // same verdict in the whole warp
        float d0[4], d1[4];
        gb_mma_bf16_1688(d0, a[0][0], a[0][1], bfrag[j]);      // positions g, g + 8
        gb_mma_bf16_1688(d1, a[1][0], a[1][1], bfrag[j]);      // positions 16 + g, 24 + g
        // v[cc][pb]: code 2t + cc of the block, position 8 pb + g
        float v[2][4] = {{d0[0], d0[2], d1[0], d1[2]}, {d0[1], d0[3], d1[1], d1[3]}};
        // Store number q of a lane takes position block (t + q) & 3, so the four lanes that share
        // g write four different bank octets: every store instruction covers all 32 banks once.
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          if (t & 1) { const float x0 = v[cc][0]; v[cc][0] = v[cc][1]; v[cc][1] = v[cc][2]; v[cc][2] = v[cc][3]; v[cc][3] = x0; }
          if (t & 2) { const float x0 = v[cc][0], x1 = v[cc][1]; v[cc][0] = v[cc][2]; v[cc][1] = v[cc][3]; v[cc][2] = x0; v[cc][3] = x1; }
          float* row = col + ((warp + j * kConsumers) * 8 + 2 * t + cc) * 64;
#pragma unroll
          for (int q = 0; q < 4; ++q) row[((t + q) & 3) * 8] = v[cc][q];
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
  // ---- stream the rows ----
  const int r = lane >> 3, lp = lane & 7, rh = r >> 1;
  uint32_t base_lo[4], base_hi[4], sel[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int j = q ^ r;                                    // this lookup's codeword of the lane's four
    base_lo[q] = tab_s + (uint32_t)rh * kRegion + (uint32_t)(4 * lp + j) * 4u;          // columns rh*2 + {0,1}
    base_hi[q] = tab_s + (uint32_t)(rh ^ 1) * kRegion + (uint32_t)(4 * lp + j) * 4u;    // the other two
    sel[q] = 0x7604u | ((uint32_t)j << 4);                  // byte 1 <- code j, bytes 0,2,3 <- the base
  }
  // lookups 0,1 fall in group r >> 1 of the lane's two, lookups 2,3 in the other
  const uint32_t sel_sc = rh ? 0x4401u : 0x4410u;
  float* my_ws = kPairs ? p.ws + ((int64_t)slice * p.P + pair) * p.N : p.ws + (int64_t)slice * p.N;
  uint16_t* my_y = nullptr;
  if constexpr (kPairs) {
    if (p.direct) my_y = pair_out_row(p, pair, p.N);
  }
  for (int st = 0; st < n_stages; ++st) {
    const int s = st % kDotStages;
    uint32_t tok;
    if (!gb_mbar_wait(&full_bar[s], (st / kDotStages) & 1, &tok)) atomicExch(p.status, 22);
    const uint32_t rowp = stage_addr(s) + (uint32_t)(4 * warp + r) * kRowBytes;
    float acc0 = 0.f, acc1 = 0.f;
    if (ns == kS) {
      // rows 0,1 of the warp take columns 0,1,2,3; rows 2,3 take 2,3,0,1
      const uint32_t pa = rowp + (uint32_t)rh * 96u, pb = rowp + (uint32_t)(rh ^ 1) * 96u;
      const uint32_t ca = pa + 4u * lp, sa = pa + 2u * lp, cb = pb + 4u * lp, sb = pb + 2u * lp;
      dot_superblock<0, 0>(ca, sa, base_lo, sel, sel_sc, tok, acc0, acc1);
      dot_superblock<48, 128>(ca, sa, base_lo, sel, sel_sc, tok, acc0, acc1);
      dot_superblock<0, 0>(cb, sb, base_hi, sel, sel_sc, tok, acc0, acc1);
      dot_superblock<48, 128>(cb, sb, base_hi, sel, sel_sc, tok, acc0, acc1);
    } else {
      // a ragged last slice: every row walks the columns in order (two-way conflicts on the
      // code and scale loads, correctness unchanged)
      uint32_t b0[4], b1[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        b0[q] = tab_s + (uint32_t)(4 * lp + (q ^ r)) * 4u;
        b1[q] = b0[q] + kRegion;
      }
      const uint32_t c0 = rowp + 4u * lp, s0 = rowp + 2u * lp;
      if (ns > 0) dot_superblock<0, 0>(c0, s0, b0, sel, sel_sc, tok, acc0, acc1);
      if (ns > 1) dot_superblock<48, 128>(c0, s0, b0, sel, sel_sc, tok, acc0, acc1);
      if (ns > 2) dot_superblock<96, 0>(c0, s0, b1, sel, sel_sc, tok, acc0, acc1);
    }
    float acc = acc0 + acc1;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    const int64_t row = row_begin + (int64_t)st * kStageRows + 4 * warp + r;
    if (lp == 0 && row < row_end) {
      if (kPairs && my_y) my_y[row] = (uint16_t)gb_f32_to_bf16_bits(acc * p.global_scale);
      else my_ws[row] = acc;
    }
    __syncwarp();
    if (lane == 0) gb_mbar_arrive(&empty_bar[s]);
  }
}

__global__ void dot_finalize_kernel(const float* __restrict__ ws, int n_slices, int64_t N, float global_scale,
                                    uint16_t* __restrict__ y) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float acc = 0.f;
  for (int s = 0; s < n_slices; ++s) acc += ws[(int64_t)s * N + n];
  y[n] = (uint16_t)gb_f32_to_bf16_bits(acc * global_scale);
}

// ---- column-parallel linear: sum the K slices and all-gather the shard in the same launch ----
// Thread i finishes outputs 2i, 2i+1 of this rank's shard, stores them at their place in this
// rank's full output row, sends the pair as one 8-byte {word, exchange number} store into every
// peer's staging slot and then collects the peers' words the same way (see gb_peer.cu for the
// flag-in-data protocol: two slot halves by parity, bounded polling, status 3 on a timeout).
struct GatherParams {
  const float* ws;
  int n_slices;
  int64_t n_local;                 // columns of this rank's shard (even)
  float global_scale;
  uint16_t* y_full;                // this rank's full output row [N]
  int n_roles;
  int lcol[4], gcol0[4], width[4]; // shard column, global column of rank 0's slice, slice width (all even)
  uint2* ll[GB_PEER_MAX];
  uint32_t* flags;                 // own flag block: [18] exchange number, [19] CTA counter
  int64_t capacity;
  int rank, world;
  int* status;
};

__global__ void __launch_bounds__(256) dot_finalize_allgather_kernel(const __grid_constant__ GatherParams p) {
  __shared__ uint32_t s_epoch;
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(p.flags + 18) + 1u;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int64_t half = (int64_t)(epoch & 1u) * p.world * p.capacity;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool late = false;
  if (2 * i < p.n_local) {
    const int64_t n = 2 * i;
    float a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < p.n_slices; ++s) {
      const float2 v = *reinterpret_cast<const float2*>(p.ws + (int64_t)s * p.n_local + n);
      a0 += v.x;
      a1 += v.y;
    }
    const uint32_t word = gb_f32_to_bf16_bits(a0 * p.global_scale) | (gb_f32_to_bf16_bits(a1 * p.global_scale) << 16);
    int r = 0;
    while (r + 1 < p.n_roles && n >= p.lcol[r + 1]) ++r;
    const int64_t off = n - p.lcol[r];                         // column inside the role's slice
    uint32_t* out32 = reinterpret_cast<uint32_t*>(p.y_full);
    out32[(p.gcol0[r] + (int64_t)p.rank * p.width[r] + off) >> 1] = word;
#pragma unroll
    for (int d = 0; d < GB_PEER_MAX; ++d)
      if (d < p.world && d != p.rank) {
        uint2* slot = p.ll[d] + half + (int64_t)p.rank * p.capacity + i;
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(slot), "r"(word), "r"(epoch) : "memory");
      }
    const uint2* slot0 = p.ll[p.rank] + half + i;
    uint2 v[GB_PEER_MAX];
#pragma unroll
    for (int src = 0; src < GB_PEER_MAX; ++src)
      if (src < p.world && src != p.rank)
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                     : "=r"(v[src].x), "=r"(v[src].y) : "l"(slot0 + (int64_t)src * p.capacity) : "memory");
#pragma unroll
    for (int src = 0; src < GB_PEER_MAX; ++src) {
      if (src >= p.world || src == p.rank) continue;
      uint64_t t0 = 0;
      for (uint32_t spin = 0; v[src].y != epoch && !late; ++spin) {
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                     : "=r"(v[src].x), "=r"(v[src].y) : "l"(slot0 + (int64_t)src * p.capacity) : "memory");
        if ((spin & 63u) == 63u) {
          const uint64_t now = gb_globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > 2000000000ull) late = true;
        }
      }
      out32[(p.gcol0[r] + (int64_t)src * p.width[r] + off) >> 1] = v[src].x;
    }
  }
  if (late) atomicExch(p.status, 3);
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(p.flags + 19, 1u);
    if (old == gridDim.x - 1) {       // every CTA has read the exchange number by now
      p.flags[19] = 0u;
      p.flags[18] = epoch;
    }
  }
}

// Pair mode: adds the K slices of every routed pair's rows, applies the global scale and, for
// the fused gate/up projection, SwiGLU with the bf16 roundings of F.silu(gate) * up
// (gridbook/native_cutlass.py:129-155), then rounds once.
__global__ void dot_pairs_finalize_kernel(const __grid_constant__ DotParams p, int swiglu) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t width = swiglu ? p.N / 2 : p.N;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)p.P * width) return;
  const int pair = (int)(i / width);
  const int64_t j = i - (int64_t)pair * width;
  const int e = p.pair_expert ? p.pair_expert[pair] - p.expert_base : 0;
  if (e < 0 || e >= p.E) return;
  float a = 0.f, b = 0.f;
  for (int s = 0; s < p.n_slices; ++s) {
    const float* slot = p.ws + ((int64_t)s * p.P + pair) * p.N;
    a += slot[j];
    if (swiglu) b += slot[j + width];
  }
  float out = a * p.global_scale;
  if (swiglu) {
    const float gate = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(out));
    const float up = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(b * p.global_scale));
    const float sl = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(gate / (1.0f + __expf(-gate))));
    out = sl * up;
  }
  pair_out_row(p, pair, width)[j] = (uint16_t)gb_f32_to_bf16_bits(out);
}

}  // namespace

int gb_prepare_dot() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemv_dot_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDotSmem));
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemv_dot_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDotSmem));
  return GB_OK;
}

int64_t gb_gemv_dot_workspace_bytes(int64_t N, int64_t K) {
  const int64_t n_slices = (K / 256 + kS - 1) / kS;
  return n_slices * N * (int64_t)sizeof(float);
}

// Launches gemv_dot_kernel<false> for one activation row; the partial sums land in `workspace`.
static int dot_launch(const void* x, const gb_weight* w, int act, int scale_rule, void* workspace,
                      int64_t workspace_bytes, cudaStream_t stream, DotParams* out) {
  const gb_format& f = w->fmt;
  const bool mine = f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
                    w->cb_row_offset == nullptr && ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0 &&
                    (act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16) && w->rows >= 256 && w->K >= 256 * kS &&
                    ((uintptr_t)x & 15u) == 0 && ((uintptr_t)w->codebook & 3u) == 0;
  if (!mine) return GB_EUNSUPPORTED;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  DotParams p = {};
  p.x = (const uint16_t*)x;
  p.codebook = (const uint16_t*)w->codebook;
  p.act = act;
  p.scale_rule = scale_rule;
  p.N = w->rows;
  p.n_sb = (int)(w->K / 256);
  p.n_slices = (p.n_sb + kS - 1) / kS;
  p.n_groups = sms / p.n_slices;
  if (p.n_groups < 1) p.n_groups = 1;
  const int64_t per = (w->rows + p.n_groups - 1) / p.n_groups;
  p.rows_per_group = (int)((per + kStageRows - 1) / kStageRows * kStageRows);
  const int64_t need = gb_gemv_dot_workspace_bytes(w->rows, w->K);
  GB_REQUIRE(workspace != nullptr && workspace_bytes >= need, "workspace of %lld bytes is too small (need %lld)",
             (long long)workspace_bytes, (long long)need);
  p.ws = (float*)workspace;
  p.status = gb_status_word();
  CUtensorMap map;
  int rc = gb_tensor_map_bytes_2d(&map, w->qw, (uint64_t)p.n_sb * 48u, (uint64_t)w->rows, (uint64_t)w->row_stride,
                                  kRowBytes, kStageRows);
  if (rc != GB_OK) return rc;
  GB_CUDA_OK(gb_launch(gemv_dot_kernel<false>, dim3(p.n_slices * p.n_groups), dim3(kDotThreads), kDotSmem, stream, map, p));
  *out = p;
  return GB_OK;
}

int gb_gemv_dot(const void* x, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  DotParams p;
  int rc = dot_launch(x, w, act, scale_rule, workspace, workspace_bytes, stream, &p);
  if (rc != GB_OK) return rc;
  const float gs = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  GB_CUDA_OK(gb_launch(dot_finalize_kernel, dim3((unsigned)((w->rows + 255) / 256)), dim3(256), 0, stream,
                       (const float*)p.ws, p.n_slices, (int64_t)w->rows, gs, (uint16_t*)y));
  return GB_OK;
}

// One activation row of a column-parallel linear: this rank's shard through the table kernel,
// then ONE launch that adds the K slices, rounds, and exchanges the shards between the ranks.
extern "C" int gb_gemv_allgather(const void* x, const gb_weight* w, int act, int scale_rule,
                                 const gb_peer_group* g, void* const* ll, int64_t ll_bytes,
                                 const gb_gather_layout* layout, void* y_full, void* workspace,
                                 int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(x && g && ll && layout && y_full, "null pointer argument");
  GB_REQUIRE(g->world >= 1 && g->world <= GB_PEER_MAX && g->rank >= 0 && g->rank < g->world, "bad peer group");
  GB_REQUIRE(layout->n_roles >= 1 && layout->n_roles <= 4, "1..4 roles, got %d", layout->n_roles);
  GatherParams q = {};
  int64_t cols = 0;
  for (int r = 0; r < layout->n_roles; ++r) {
    GB_REQUIRE(layout->width[r] > 0 && layout->width[r] % 2 == 0 && layout->gcol0[r] % 2 == 0 && layout->lcol[r] == cols,
               "role %d: slices must be even, contiguous in the shard and start on even columns", r);
    q.lcol[r] = (int)layout->lcol[r];
    q.gcol0[r] = (int)layout->gcol0[r];
    q.width[r] = (int)layout->width[r];
    cols += layout->width[r];
  }
  GB_REQUIRE(cols == w->rows, "the roles cover %lld columns, the shard has %lld rows", (long long)cols, (long long)w->rows);
  GB_REQUIRE(((uintptr_t)y_full & 3u) == 0, "output must be 4-byte aligned");
  q.capacity = ll_bytes / (2 * (int64_t)g->world * 8);
  if (cols / 2 > q.capacity) return GB_EUNSUPPORTED;      // staging buffer too small: take the two-launch route
  for (int r = 0; r < g->world; ++r) {
    GB_REQUIRE(ll[r] != nullptr && g->flags[r] != nullptr, "peer buffers of rank %d missing", r);
    q.ll[r] = (uint2*)ll[r];
  }
  DotParams p;
  rc = dot_launch(x, w, act, scale_rule, workspace, workspace_bytes, stream, &p);
  if (rc != GB_OK) return rc;           // GB_EUNSUPPORTED: the caller runs gb_gemv + gb_peer_allgather_ll
  q.ws = p.ws;
  q.n_slices = p.n_slices;
  q.n_local = w->rows;
  q.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  q.y_full = (uint16_t*)y_full;
  q.n_roles = layout->n_roles;
  q.flags = (uint32_t*)g->flags[g->rank];
  q.rank = g->rank;
  q.world = g->world;
  q.status = gb_status_word();
  GB_CUDA_OK(gb_launch(dot_finalize_allgather_kernel, dim3((unsigned)((cols / 2 + 255) / 256)), dim3(256), 0, stream, q));
  return GB_OK;
}

// ---------------------------------------------------------------------------
// Routed layer, small batches: every (token, expert) pair is its own M = 1 linear through the
// table kernel above.  An expert's weights stream once per PAIR (as in the reference's grouped
// GEMV, gridbook/csrc/cb_gemv.cu:1220-1233), so this pays while few pairs share an expert.
// ---------------------------------------------------------------------------
extern "C" int64_t gb_moe_gemv_pairs_workspace_bytes(int64_t P, int64_t rows, int64_t K) {
  const int64_t n_slices = (K / 256 + kS - 1) / kS;
  return n_slices * P * rows * (int64_t)sizeof(float);
}

struct PairChain {            // set for the second projection of gb_moe_mlp_pairs
  const float* xws;
  int slices;
  int64_t N;
  float scale;
};
static int dot_pairs_launch(const void* x, const int32_t* x_row, const gb_weight* w, int64_t expert_stride,
                            int64_t E, int64_t expert_base, const int32_t* pair_expert, int64_t P,
                            int64_t pairs_expected, int swiglu, int act, int scale_rule, void* y,
                            const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes, void* stream_,
                            bool leave_partials = false, const PairChain* chain = nullptr);

extern "C" int gb_moe_gemv_pairs(const void* x, const int32_t* x_row, const gb_weight* w, int64_t expert_stride,
                                 int64_t E, int64_t expert_base, const int32_t* pair_expert, int64_t P,
                                 int64_t pairs_expected, int swiglu, int act, int scale_rule, void* y,
                                 const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes, void* stream_) {
  GB_REQUIRE(pair_expert != nullptr, "null pair_expert");
  return dot_pairs_launch(x, x_row, w, expert_stride, E, expert_base, pair_expert, P, pairs_expected, swiglu, act,
                          scale_rule, y, y_rows, workspace, workspace_bytes, stream_);
}

// A few activation rows against ONE matrix: row m is "pair" m of a one-expert stack, so the
// weights stream once per row (the second and later passes mostly out of L2).  Worth it while
// that beats expanding every weight for the MMA kernel; the caller decides up to which M.
int gb_gemv_dot_rows(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                     int64_t workspace_bytes, void* stream_) {
  if (w->rows < 256) return GB_EUNSUPPORTED;
  return dot_pairs_launch(x, nullptr, w, w->rows * w->row_stride, 1, 0, nullptr, M, 0, 0, act, scale_rule, y, nullptr,
                          workspace, workspace_bytes, stream_);
}

int64_t gb_gemv_dot_rows_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  return gb_moe_gemv_pairs_workspace_bytes(M, N, K);
}

static int dot_pairs_launch(const void* x, const int32_t* x_row, const gb_weight* w, int64_t expert_stride,
                            int64_t E, int64_t expert_base, const int32_t* pair_expert, int64_t P,
                            int64_t pairs_expected, int swiglu, int act, int scale_rule, void* y,
                            const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes, void* stream_,
                            bool leave_partials, const PairChain* chain) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  GB_REQUIRE((x || chain) && (y || y_rows || leave_partials), "null pointer argument");
  GB_REQUIRE(E >= 1 && P >= 0 && P < (1 << 24), "bad E=%lld P=%lld", (long long)E, (long long)P);
  GB_REQUIRE(!swiglu || w->rows % 2 == 0, "swiglu needs an even row count");
  const gb_format& f = w->fmt;
  const bool mine = f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
                    w->cb_row_offset == nullptr && ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0 &&
                    expert_stride == w->rows * w->row_stride && E * w->rows < (1ll << 31) &&
                    (act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16) && w->K >= 256 &&
                    ((uintptr_t)x & 15u) == 0 && ((uintptr_t)w->codebook & 3u) == 0;
  if (!mine) return GB_EUNSUPPORTED;
  if (P == 0) return GB_OK;
  if (chain) GB_REQUIRE(chain->xws && chain->N == 2 * w->K, "chained input must be a gate/up projection of 2 x K rows");
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  DotParams p = {};
  p.x = (const uint16_t*)x;
  p.x_row = x_row;
  p.codebook = (const uint16_t*)w->codebook;
  p.act = act;
  p.scale_rule = scale_rule;
  p.N = w->rows;
  p.n_sb = (int)(w->K / 256);
  p.n_slices = (p.n_sb + kS - 1) / kS;
  p.pair_expert = pair_expert;
  p.P = (int)P;
  p.E = (int)E;
  p.expert_base = (int)expert_base;
  p.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  p.status = gb_status_word();
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
  // row bands per pair: enough CTAs to cover the machine with the pairs expected to be live here
  int64_t live = pairs_expected > 0 && pairs_expected < P ? pairs_expected : P;
  int bands = (int)(sms / (live * p.n_slices));
  const int max_bands = (int)((w->rows + kStageRows - 1) / kStageRows);
  if (bands > max_bands) bands = max_bands;
  if (bands < 1) bands = 1;
  p.bands = bands;
  const int64_t per = (w->rows + bands - 1) / bands;
  p.rows_per_group = (int)((per + kStageRows - 1) / kStageRows * kStageRows);
  p.direct = (p.n_slices == 1 && !swiglu && !leave_partials) ? 1 : 0;
  if (chain) {
    p.xws = chain->xws;
    p.xws_slices = chain->slices;
    p.xws_N = chain->N;
    p.xws_scale = chain->scale;
  }
  if (!p.direct) {
    const int64_t need = gb_moe_gemv_pairs_workspace_bytes(P, w->rows, w->K);
    GB_REQUIRE(workspace != nullptr && workspace_bytes >= need, "workspace of %lld bytes is too small (need %lld)",
               (long long)workspace_bytes, (long long)need);
    p.ws = (float*)workspace;
  }
  CUtensorMap map;
  rc = gb_tensor_map_bytes_2d(&map, w->qw, (uint64_t)p.n_sb * 48u, (uint64_t)(E * w->rows), (uint64_t)w->row_stride,
                              kRowBytes, kStageRows);
  if (rc != GB_OK) return rc;
  const int64_t grid = P * p.n_slices * bands;
  GB_REQUIRE(grid < (1ll << 31), "too many pairs for one launch");
  GB_CUDA_OK(gb_launch(gemv_dot_kernel<true>, dim3((unsigned)grid), dim3(kDotThreads), kDotSmem, stream, map, p));
  if (!p.direct && !leave_partials) {
    const int64_t total = P * (swiglu ? w->rows / 2 : w->rows);
    GB_CUDA_OK(gb_launch(dot_pairs_finalize_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, p,
                         swiglu ? 1 : 0));
  }
  return GB_OK;
}

// Both projections of the routed MLP for small batches, in two launches: the gate/up table
// GEMVs leave their K-slice partial sums in the workspace, and the down projection's kernels
// sum them, apply SwiGLU and the fp4 bucket while they stage their activation row.
extern "C" int64_t gb_moe_mlp_pairs_workspace_bytes(int64_t P, int64_t hidden, int64_t inter) {
  return gb_moe_gemv_pairs_workspace_bytes(P, 2 * inter, hidden) + gb_moe_gemv_pairs_workspace_bytes(P, hidden, inter);
}

extern "C" int gb_moe_mlp_pairs(const void* x, const int32_t* x_row, const gb_weight* w13, int64_t stride13,
                                const gb_weight* w2, int64_t stride2, int64_t E, int64_t expert_base,
                                const int32_t* pair_expert, int64_t P, int64_t pairs_expected, int act, int scale_rule,
                                void* y, const gb_peer_rows* y_rows, void* workspace, int64_t workspace_bytes,
                                void* stream) {
  GB_REQUIRE(w13 && w2 && pair_expert, "null pointer argument");
  GB_REQUIRE(w13->rows == 2 * w2->K && w2->rows == w13->K, "gate/up is %lld x %lld, down %lld x %lld: not an MLP",
             (long long)w13->rows, (long long)w13->K, (long long)w2->rows, (long long)w2->K);
  const int64_t ws13 = gb_moe_gemv_pairs_workspace_bytes(P, w13->rows, w13->K);
  GB_REQUIRE(workspace && workspace_bytes >= gb_moe_mlp_pairs_workspace_bytes(P, w13->K, w2->K),
             "workspace of %lld bytes is too small", (long long)workspace_bytes);
  int rc = dot_pairs_launch(x, x_row, w13, stride13, E, expert_base, pair_expert, P, pairs_expected, 0, act, scale_rule,
                            nullptr, nullptr, workspace, ws13, stream, /*leave_partials=*/true, nullptr);
  if (rc != GB_OK) return rc;
  PairChain chain;
  chain.xws = (const float*)workspace;
  chain.slices = (int)((w13->K / 256 + kS - 1) / kS);
  chain.N = w13->rows;
  chain.scale = w13->global_scale == 0.0f ? 1.0f : w13->global_scale;
  return dot_pairs_launch(nullptr, nullptr, w2, stride2, E, expert_base, pair_expert, P, pairs_expected, 0, act,
                          scale_rule, y, y_rows, (uint8_t*)workspace + ws13, workspace_bytes - ws13, stream, false, &chain);
}
