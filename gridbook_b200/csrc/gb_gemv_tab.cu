// One activation row of the literal format (fp4 grid, full mode, k = 8, E4M3-direct scales)
// against one matrix, or against several matrices that read the same row (q and kv of an
// attention block, gate and up of an MLP), in ONE launch.
//
// The arithmetic is the inner-product-table formulation of gb_gemv_dot.cu: a CTA owns four
// superblock columns of K and a band of rows, builds T[s][c][v] = <codebook[c], x[256 s + 8 v ..+8]>
// for its columns (tensor cores, 128 KiB of fp32 in shared memory) and streams its rows through a
// TMA ring; a weight costs a table lookup instead of a decode.  What differs:
//
//   * Four lanes walk one row (eight codewords each), so a warp takes eight rows per pass: the code
//     and scale loads, the barrier traffic and the cross-lane sum are shared by twice the bytes.
//   * The table is built with the codewords on the M side of the MMA, so a thread ends up with
//     eight neighbouring positions of one codeword and writes them with two 16-byte stores.
//   * The K-slice partial sums are not added by a second kernel.  Every (slice, row) partial sum
//     goes to its own slot of an "armed" buffer - one whose every word reads 0xFFFFFFFF, a NaN
//     pattern no arithmetic here can produce - and the CTAs of a band share the band's rows
//     between them: each polls the slots of its share until they hold a value, adds them in
//     slice order, rounds once to bf16, and re-arms the slots.  The data is its own flag, so the
//     tail of a linear is one store, one poll and one store, with no fence, no counter and no
//     second launch, and the result does not depend on the order in which CTAs finish.
//
// All CTAs of a launch must be able to run at the same time (a CTA that polls holds its SM), so
// the grid never exceeds the number of SMs; every wait is bounded and raises the status word.
#include "gb_common.cuh"

#include <cuda.h>

namespace {

constexpr int kS = 4;                           // superblock columns per CTA
constexpr int kWarps = 16;                      // consumer warps; warps 0-7 take even stages, 8-15 odd ones
constexpr int kThreads = (kWarps + 1) * 32;
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kStageRows = 64;                  // eight rows for each of the eight warps of a group
constexpr int kBoxBytes = kStageRows * 96;      // one TMA box: two columns (96 bytes) of 64 rows
constexpr int kStageBytes = 2 * kBoxBytes;
constexpr int kStages = 6;
constexpr int kFront = 5;                       // ring stages in front of the tables, the last one behind
constexpr uint32_t kTab0 = 0x10000u;            // shared-window address of the tables (a multiple of 64 KiB)
constexpr uint32_t kRegion = 0x10000u;          // 256 codewords x 256-byte rows: columns {0,1}, then {2,3}
constexpr uint32_t kBack0 = kTab0 + 2u * kRegion;
constexpr int kSmem = (int)(kBack0 + kStageBytes);
constexpr uint32_t kEmpty = 0xFFFFFFFFu;
constexpr int kMaxSeg = 4;
constexpr int kHeaderBytes = 256;               // head of the armed buffer: never written, checked as a canary

struct TabSeg {
  const uint16_t* codebook;     // [256 * 8] bf16
  uint16_t* y;                  // [N] bf16
  float* slots;                 // [n_slices][N], armed
  int64_t N;
  int rows_per_band, band0, bands, lanes_per_row;
  float global_scale;
};

struct TabParams {
  const uint16_t* x;            // [K] bf16
  const uint32_t* canary;
  int* status;
  unsigned long long wait_ns;
  int act, scale_rule, n_sb, n_slices, n_seg;
  TabSeg seg[kMaxSeg];
};

struct TabMaps {
  CUtensorMap m[kMaxSeg];
};

// Shared-memory loads that carry the token of the barrier wait that made the data visible: free
// to be reordered among themselves, never above that wait.
template <int kImm>
GB_DEVINL float lds_f32(uint32_t a, uint32_t tok) {
  float v;
  asm("ld.shared.f32 %0, [%1+%2]; // %3" : "=f"(v) : "r"(a), "n"(kImm), "r"(tok));
  return v;
}
template <int kImm>
GB_DEVINL uint32_t lds_u32(uint32_t a, uint32_t tok) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2]; // %3" : "=r"(v) : "r"(a), "n"(kImm), "r"(tok));
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
GB_DEVINL void sts_v4(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
GB_DEVINL uint32_t ld_slot(const float* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
GB_DEVINL void st_slot(float* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One superblock column of one row for this lane's eight codewords (four groups).  pA / pB point
// at the lane's two code words inside column 0 of the row, pS at its four scale bytes.
template <int kCol>
GB_DEVINL void tab_column(uint32_t pA, uint32_t pB, uint32_t pS, const uint32_t (&base)[8], const uint32_t (&sel)[4],
                          uint32_t selsc, uint32_t tok, float& acc0, float& acc1) {
  constexpr int kBox = (kCol >> 1) * kBoxBytes + (kCol & 1) * 48;
  constexpr int kTab = (int)(kTab0 + (uint32_t)(kCol >> 1) * kRegion + (uint32_t)(kCol & 1) * 128u);
  const uint32_t cA = lds_u32<kBox>(pA, tok);
  const uint32_t cB = lds_u32<kBox>(pB, tok);
  const uint32_t sc = lds_u32<kBox + 32>(pS, tok);
  const float t0 = lds_f32<kTab>(__byte_perm(cA, base[0], sel[0]), tok);
  const float t1 = lds_f32<kTab>(__byte_perm(cA, base[1], sel[1]), tok);
  const float t2 = lds_f32<kTab>(__byte_perm(cA, base[2], sel[2]), tok);
  const float t3 = lds_f32<kTab>(__byte_perm(cA, base[3], sel[3]), tok);
  const float t4 = lds_f32<kTab>(__byte_perm(cB, base[4], sel[0]), tok);
  const float t5 = lds_f32<kTab>(__byte_perm(cB, base[5], sel[1]), tok);
  const float t6 = lds_f32<kTab>(__byte_perm(cB, base[6], sel[2]), tok);
  const float t7 = lds_f32<kTab>(__byte_perm(cB, base[7], sel[3]), tok);
  const uint32_t scp = __byte_perm(sc, 0u, selsc);        // byte m: the scale of lookups 2m, 2m+1
  float f0, f1, f2, f3;
  e4m3x2_to_f32(scp, f0, f1);
  e4m3x2_to_f32(scp >> 16, f2, f3);
  acc0 = fmaf(t0 + t1, f0, acc0);
  acc1 = fmaf(t2 + t3, f1, acc1);
  acc0 = fmaf(t4 + t5, f2, acc0);
  acc1 = fmaf(t6 + t7, f3, acc1);
}

__global__ void __launch_bounds__(kThreads, 1)
gemv_tab_kernel(const __grid_constant__ TabMaps maps, const __grid_constant__ TabParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base_s = gb_smem_u32(smem);
  const uint32_t front_s = (base_s + 127u) & ~127u;
  const uint32_t xq_s = front_s + kFront * kStageBytes;
  const uint32_t bar_s = xq_s + kS * 512;
  if (bar_s + 2 * kStages * 8 > kTab0) {          // same verdict in every thread, before any barrier
    if (threadIdx.x == 0) atomicExch(p.status, 23);
    return;
  }
  uint32_t* xq = reinterpret_cast<uint32_t*>(smem + (xq_s - base_s));       // kS * 256 bf16
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (bar_s - base_s));
  uint64_t* empty_bar = full_bar + kStages;
  auto stage_addr = [&](int s) -> uint32_t { return s < kFront ? front_s + (uint32_t)s * kStageBytes : kBack0; };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x % p.n_slices;
  int band = blockIdx.x / p.n_slices;
  int si = 0;
  while (si + 1 < p.n_seg && band >= p.seg[si + 1].band0) ++si;
  const TabSeg& sg = p.seg[si];
  band -= sg.band0;
  const int sb0 = slice * kS;
  const int ns = min(kS, p.n_sb - sb0);
  const int64_t row_begin = (int64_t)band * sg.rows_per_band;
  const int64_t row_end = min(sg.N, row_begin + sg.rows_per_band);
  if (row_end <= row_begin) return;
  const int n_stages = (int)((row_end - row_begin + kStageRows - 1) / kStageRows);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      gb_mbar_init(&full_bar[s], 1);
      gb_mbar_init(&empty_bar[s], kWarps / 2);
    }
    gb_fence_barrier_init();
  }
  __syncthreads();
  gb_pdl_launch_dependents();

  if (warp == kWarps) {
    // ------------------------------ producer ------------------------------
    // The weight stream depends on nothing an earlier kernel wrote: the ring fills while the
    // kernel before this one is still finishing.
    if (lane == 0) {
      const uint64_t map = reinterpret_cast<uint64_t>(&maps.m[si]);
      const uint32_t tx = ns > 2 ? kStageBytes : kBoxBytes;
      for (int st = 0; st < n_stages; ++st) {
        const int s = st % kStages;
        if (!gb_mbar_wait(&empty_bar[s], ((st / kStages) & 1) ^ 1)) {
          gb_pdl_wait();
          atomicExch(p.status, 21);
          break;
        }
        gb_mbar_expect_tx(&full_bar[s], tx);
        const int row = (int)(row_begin + (int64_t)st * kStageRows);
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(stage_addr(s)), "l"(map), "r"(sb0 * 48), "r"(row), "r"(gb_smem_u32(&full_bar[s]))
            : "memory");
        if (ns > 2)
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
              ::"r"(stage_addr(s) + kBoxBytes), "l"(map), "r"(sb0 * 48 + 96), "r"(row), "r"(gb_smem_u32(&full_bar[s]))
              : "memory");
      }
    }
    return;
  }

  // ---- this warp's sixteen codewords as the A fragment of the table MMAs (before the wait) ----
  const int g = lane >> 2, t = lane & 3;
  uint32_t a0, a1;
  {
    const uint32_t* cb32 = reinterpret_cast<const uint32_t*>(sg.codebook);
    a0 = __ldg(cb32 + (16 * warp + g) * 4 + t);
    a1 = __ldg(cb32 + (16 * warp + g + 8) * 4 + t);
  }

  // ---- lane constants of the row stream (nothing here depends on an earlier kernel) ----
  // Lane (r, lp): row r of the warp's eight, codewords 8 lp .. 8 lp + 7 of every column.  Lookup q
  // of a lane is its codeword q ^ r, so the 32 lanes of a lookup read 32 different positions =
  // banks.  The lane's two code words are loaded separately (rows 0-3 take their low word first,
  // rows 4-7 their high word), which makes those loads conflict-free as well.
  const int r = lane >> 2, lp = lane & 3;
  uint32_t base[8], sel[4], selsc = 0;
#pragma unroll
  for (int q = 0; q < 8; ++q) base[q] = (uint32_t)(8 * lp + (q ^ r)) * 4u;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    sel[q] = 0x7604u | ((uint32_t)((q ^ r) & 3) << 4);     // byte 1 <- that code byte, bytes 0,2,3 <- the base
    selsc |= (uint32_t)(q ^ (r >> 1)) << (4 * q);          // lookups 2q, 2q+1 lie in group q ^ (r >> 1) of the lane's four
  }

  // ---- this slice of the activation row, through its bucket, into shared memory ----
  gb_pdl_wait();                       // the activations and the slots belong to earlier kernels
  if (blockIdx.x == 0 && tid == 0 && ld_slot(reinterpret_cast<const float*>(p.canary)) != kEmpty)
    atomicExch(p.status, 24);          // the slot buffer was never armed: the sums of this call are void
  if (tid < ns * 128) {                // two values per thread, a bucket group per eight lanes
    uint32_t w = reinterpret_cast<const uint32_t*>(p.x + (int64_t)sb0 * 256)[tid];
    if (p.act == GB_ACT_FP4_GROUP16) w = gb_fp4_group16_qdq_lanes(w, p.scale_rule);
    // word (position, k pair kp) of a column is kept at [kp][(position + 8 kp) mod 32]: the four
    // positions a thread feeds to its four table MMAs are one 16-byte load, free of bank conflicts
    const int wi = tid & 127, kp = wi & 3, pos = wi >> 2;
    xq[(tid & ~127) + 32 * kp + ((pos + 8 * kp) & 31)] = w;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");

  // ---- inner-product tables ----
  // Per column four MMAs with this warp's codewords as the 16 rows and eight positions as the
  // columns.  Column n of MMA nb is position 8 (n >> 1) + 4 (n & 1) + nb, which leaves thread
  // (g, t) with positions 8 t .. 8 t + 7 of codewords g and g + 8: two 16-byte stores each.  Odd g
  // stores its upper half first, so the two rows of a quarter-warp fill all 32 banks.
#pragma unroll
  for (int s = 0; s < kS; ++s) {
    if (s >= ns) break;
    const uint4 b = *reinterpret_cast<const uint4*>(xq + s * 128 + 32 * t + ((8 * (g >> 1) + 4 * (g & 1) + 8 * t) & 31));
    float d[4][4];
    gb_mma_bf16_1688(d[0], a0, a1, b.x);
    gb_mma_bf16_1688(d[1], a0, a1, b.y);
    gb_mma_bf16_1688(d[2], a0, a1, b.z);
    gb_mma_bf16_1688(d[3], a0, a1, b.w);
    // d[nb][e]: codeword g, position 8 t + 4 e + nb;  d[nb][2 + e]: codeword g + 8
    const uint32_t row_lo = kTab0 + (uint32_t)(s >> 1) * kRegion + (uint32_t)(16 * warp + g) * 256u +
                            (uint32_t)(s & 1) * 128u + 32u * (uint32_t)t;
    const uint32_t row_hi = row_lo + 8u * 256u;
    const bool odd = (g & 1) != 0;
    const uint32_t o1 = odd ? 16u : 0u, o2 = 16u - o1;
    sts_v4(row_lo + o1, odd ? d[0][1] : d[0][0], odd ? d[1][1] : d[1][0], odd ? d[2][1] : d[2][0], odd ? d[3][1] : d[3][0]);
    sts_v4(row_hi + o1, odd ? d[0][3] : d[0][2], odd ? d[1][3] : d[1][2], odd ? d[2][3] : d[2][2], odd ? d[3][3] : d[3][2]);
    sts_v4(row_lo + o2, odd ? d[0][0] : d[0][1], odd ? d[1][0] : d[1][1], odd ? d[2][0] : d[2][1], odd ? d[3][0] : d[3][1]);
    sts_v4(row_hi + o2, odd ? d[0][2] : d[0][3], odd ? d[1][2] : d[1][3], odd ? d[2][2] : d[2][3], odd ? d[3][2] : d[3][3]);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");

  // ---- stream the rows ----
  const int grp = warp >> 3, wl = warp & 7;
  float* my_slots = sg.slots + (int64_t)slice * sg.N;
  for (int st = grp; st < n_stages; st += 2) {
    const int s = st % kStages;
    uint32_t tok;
    if (!gb_mbar_wait(&full_bar[s], (st / kStages) & 1, &tok)) {
      atomicExch(p.status, 22);
      break;
    }
    const uint32_t rowp = stage_addr(s) + (uint32_t)(wl * 8 + r) * 96u;
    const uint32_t pA = rowp + 8u * lp + 4u * (uint32_t)(r >> 2), pB = rowp + 8u * lp + 4u * (uint32_t)(1 - (r >> 2));
    const uint32_t pS = rowp + 4u * lp;
    float acc0 = 0.f, acc1 = 0.f;
    if (ns == kS) {
      tab_column<0>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
      tab_column<1>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
      tab_column<2>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
      tab_column<3>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
    } else {                          // a ragged last slice: only the columns that exist have a table
      tab_column<0>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
      if (ns > 1) tab_column<1>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
      if (ns > 2) tab_column<2>(pA, pB, pS, base, sel, selsc, tok, acc0, acc1);
    }
    float acc = acc0 + acc1;
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    const int64_t row = row_begin + (int64_t)st * kStageRows + wl * 8 + r;
    if (lp == 0 && row < row_end) st_slot(my_slots + row, __float_as_uint(acc));
    __syncwarp();
    if (lane == 0) gb_mbar_arrive(&empty_bar[s]);
  }

  // ---- finish this CTA's share of the band: rows [m0, m1), every slice's slot ----
  // lanes_per_row lanes share a row's slices (lane j takes slices j, j + L, ...); a fixed shuffle
  // tree adds the lanes' sums, so the order of the additions never changes from run to run.
  const int L = sg.lanes_per_row;
  const int64_t share = (row_end - row_begin + p.n_slices - 1) / p.n_slices;
  const int64_t m0 = row_begin + (int64_t)slice * share;
  const int64_t m1 = min(row_end, m0 + share);
  const int rows_per_iter = kConsumerThreads / L;
  const int sub = tid & (L - 1);
  const int iters = m1 > m0 ? (int)((m1 - m0 + rows_per_iter - 1) / rows_per_iter) : 0;
  bool late = false;
  for (int it = 0; it < iters; ++it) {
    const int64_t row = m0 + (int64_t)it * rows_per_iter + tid / L;
    const bool valid = row < m1;
    float sum = 0.f;
    if (valid) {
      for (int sl0 = sub; sl0 < p.n_slices; sl0 += 8 * L) {
        uint32_t v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int sl = sl0 + i * L;
          v[i] = sl < p.n_slices ? ld_slot(sg.slots + (int64_t)sl * sg.N + row) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int sl = sl0 + i * L;
          if (sl >= p.n_slices) break;
          float* slot = sg.slots + (int64_t)sl * sg.N + row;
          uint64_t t0 = 0;
          for (uint32_t spin = 0; v[i] == kEmpty && !late; ++spin) {
            v[i] = ld_slot(slot);
            if ((spin & 63u) == 63u) {
              const uint64_t now = gb_globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > p.wait_ns) late = true;
            }
          }
          sum += __uint_as_float(v[i]);
          st_slot(slot, kEmpty);
        }
      }
    }
    for (int o = 1; o < L; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (valid && sub == 0) sg.y[row] = (uint16_t)gb_f32_to_bf16_bits(sum * sg.global_scale);
  }
  if (late) atomicExch(p.status, 25);
}

bool tab_serves(const gb_weight* w) {
  const gb_format& f = w->fmt;
  return f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
         w->cb_row_offset == nullptr && ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0 &&
         ((uintptr_t)w->codebook & 3u) == 0 && w->rows >= kStageRows;
}

int64_t seg_slot_bytes(int64_t rows, int64_t K) {
  const int64_t n_slices = (K / 256 + kS - 1) / kS;
  return (n_slices * rows * (int64_t)sizeof(float) + 255) & ~255ll;
}

}  // namespace

int gb_prepare_tab() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemv_tab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  return GB_OK;
}

extern "C" {

int64_t gb_gemv_tab_slots_bytes(const gb_weight* const* w, int n_weights) {
  if (w == nullptr || n_weights < 1 || n_weights > kMaxSeg) return 0;
  int64_t total = kHeaderBytes;
  for (int i = 0; i < n_weights; ++i) {
    if (w[i] == nullptr || w[i]->K <= 0 || w[i]->rows <= 0) return 0;
    total += seg_slot_bytes(w[i]->rows, w[i]->K);
  }
  return total;
}

int gb_gemv_tab_arm(void* slots, int64_t bytes, void* stream) {
  GB_REQUIRE(slots != nullptr && bytes >= kHeaderBytes, "null or undersized slot buffer");
  GB_CUDA_OK(cudaMemsetAsync(slots, 0xFF, (size_t)bytes, (cudaStream_t)stream));
  return GB_OK;
}

int gb_gemv_tab(const void* x, const gb_weight* const* w, void* const* y, int n_weights, int act, int scale_rule,
                void* slots, int64_t slots_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  GB_REQUIRE(x && w && y && slots, "null pointer argument");
  GB_REQUIRE(n_weights >= 1 && n_weights <= kMaxSeg, "1..%d matrices per call, got %d", kMaxSeg, n_weights);
  GB_REQUIRE(act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16, "the table kernel fuses the fp4 group-16 bucket only (act %d)", act);
  int64_t sum_rows = 0;
  for (int i = 0; i < n_weights; ++i) {
    int rc = gb_check_weight(w[i]);
    if (rc != GB_OK) return rc;
    GB_REQUIRE(y[i] != nullptr, "null output %d", i);
    GB_REQUIRE(w[i]->K == w[0]->K, "matrix %d has K=%lld, matrix 0 K=%lld: they must read the same row", i,
               (long long)w[i]->K, (long long)w[0]->K);
    if (!tab_serves(w[i])) return GB_EUNSUPPORTED;
    sum_rows += w[i]->rows;
  }
  if (((uintptr_t)x & 3u) != 0) return GB_EUNSUPPORTED;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  const int64_t need = gb_gemv_tab_slots_bytes(w, n_weights);
  GB_REQUIRE(slots_bytes >= need && ((uintptr_t)slots & 255u) == 0,
             "slot buffer of %lld bytes is too small or not 256-byte aligned (need %lld)", (long long)slots_bytes,
             (long long)need);

  TabParams p = {};
  TabMaps maps;
  p.x = (const uint16_t*)x;
  p.canary = (const uint32_t*)slots;
  p.status = gb_status_word();
  p.wait_ns = gb_wait_limit_ns();
  p.act = act;
  p.scale_rule = scale_rule;
  p.n_sb = (int)(w[0]->K / 256);
  p.n_slices = (p.n_sb + kS - 1) / kS;
  p.n_seg = n_weights;
  // Row bands: as many as fit one CTA per SM, shared out by row count (every matrix at least one).
  int total = sms / p.n_slices;
  if (total < n_weights) return GB_EUNSUPPORTED;          // K too wide for one wave of CTAs
  int bands[kMaxSeg], used = 0;
  for (int i = 0; i < n_weights; ++i) {
    bands[i] = (int)((int64_t)total * w[i]->rows / sum_rows);
    if (bands[i] < 1) bands[i] = 1;
    used += bands[i];
  }
  auto rows_per = [&](int i) { return (double)w[i]->rows / bands[i]; };
  while (used != total) {                                 // hand out (or take back) bands where it evens the load most
    int pick = -1;
    for (int i = 0; i < n_weights; ++i) {
      if (used > total && bands[i] <= 1) continue;
      if (pick < 0 || (used < total ? rows_per(i) > rows_per(pick) : rows_per(i) < rows_per(pick))) pick = i;
    }
    if (pick < 0) return GB_EUNSUPPORTED;
    bands[pick] += used < total ? 1 : -1;
    used += used < total ? 1 : -1;
  }
  uint8_t* slot_ptr = (uint8_t*)slots + kHeaderBytes;
  int band0 = 0;
  for (int i = 0; i < n_weights; ++i) {
    TabSeg& s = p.seg[i];
    s.codebook = (const uint16_t*)w[i]->codebook;
    s.y = (uint16_t*)y[i];
    s.slots = (float*)slot_ptr;
    slot_ptr += seg_slot_bytes(w[i]->rows, w[i]->K);
    s.N = w[i]->rows;
    const int64_t per = (w[i]->rows + bands[i] - 1) / bands[i];
    s.rows_per_band = (int)((per + kStageRows - 1) / kStageRows * kStageRows);
    s.bands = (int)((w[i]->rows + s.rows_per_band - 1) / s.rows_per_band);
    s.band0 = band0;
    band0 += s.bands;
    const int share = (s.rows_per_band + p.n_slices - 1) / p.n_slices;
    int L = 1;
    while (L < 32 && L < p.n_slices && share * 2 * L <= kConsumerThreads) L *= 2;
    s.lanes_per_row = L;
    s.global_scale = w[i]->global_scale == 0.0f ? 1.0f : w[i]->global_scale;
    int rc = gb_tensor_map_bytes_2d(&maps.m[i], w[i]->qw, (uint64_t)p.n_sb * 48u, (uint64_t)w[i]->rows,
                                    (uint64_t)w[i]->row_stride, 96, kStageRows);
    if (rc != GB_OK) return rc;
  }
  for (int i = n_weights; i < kMaxSeg; ++i) maps.m[i] = maps.m[0];
  GB_CUDA_OK(gb_launch(gemv_tab_kernel, dim3((unsigned)(p.n_slices * band0)), dim3(kThreads), kSmem, stream, maps, p));
  return GB_OK;
}

}  // extern "C"
