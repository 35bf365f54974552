// Decode-batch linear on the tensor cores, without a decoded copy in HBM or in shared memory:
// y[M, N] = x[M, K] . W^T for 1 <= M <= 128 activation rows.
//
// The WEIGHTS are the M side of the MMA and live in TENSOR MEMORY: a CTA owns 128 weight rows and
// a K slice.  One warp streams the packed rows into shared memory with tiled TMA loads, one warp
// streams the matching 64-wide K slabs of the (bucketed) activations with the 128-byte swizzle,
// sixteen warps decode.  A decoder thread owns ONE weight row (= its tensor-memory lane): it reads
// the row's bytes of a superblock with 16-byte loads (rows are an odd number of 16-byte units apart
// in shared memory, so eight neighbouring rows hit eight bank groups) and per codeword its
// codebook entries from copies that are replicated so that the lanes of a load phase never share
// a bank; the decode contract's bf16(value * scale) is one packed bf16 multiply where both factors
// are exact in bf16 (fp4 grid) and an fp32 multiply + one rounding otherwise (fp8 grid); sixteen
// decoded bf16 pairs go to the lane's columns with one tcgen05.st.  One thread per operand buffer
// issues tcgen05.mma (A from tensor memory, M = 128 weight rows, N = activation rows padded to 16,
// kind::f16) into its own fp32 accumulator, which lives in tensor memory too and never leaves it
// during the K loop.  Four warpgroups of decoders, one per operand buffer (half a superblock of K,
// 64 columns), take the units in turn, so decoding, the MMAs of the units before and the loads
// overlap.  The decoders read the accumulators out at the end (lane = weight row, column =
// activation row), add them and store bf16, or fp32 partial sums per K slice that a small second
// kernel adds (summing them in the last CTA of a tile to arrive instead was measured: slower from
// 16 rows on - one CTA's serial L2 reads against a launch that uses the whole GPU).
//
// Four packed formats: the literal one (fp4 grid, full k = 8, E4M3 scale bytes: 48-byte
// superblocks), the two-tier product format fp4 k = 16 with its superblocks padded from 73 to 80
// bytes (so that rows can be fetched by TMA), and the fp8 product format k = 32 (128 bytes).
#include "gb_common.cuh"

#include <cuda.h>

namespace {

constexpr int kBM = 128;                                  // weight rows per CTA
constexpr int kDecWarps = 16;                             // four warpgroups, one per operand buffer
constexpr int kCtlWarps = 6;                              // raw producer, x producer, four MMA issuers
constexpr int kUmmaThreads = 32 * (kCtlWarps + kDecWarps);
constexpr int kMaxRows = 128;                             // activation rows
constexpr int kABufCols = 64;                             // half a superblock: 128 weights of K as bf16 pairs
constexpr uint32_t kACol0 = 256;                          // columns [0, 256): one accumulator per MMA issuer
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxXStages = 8;
constexpr int kMaxRawStages = 3;
constexpr int kSmemCap = 227 * 1024;

enum { kFmtLit = 0, kFmtK16 = 1, kFmtFp8 = 2, kFmtF8L = 3 };

// Per format: bytes of a superblock, how a raw stage is cut into TMA boxes, ring depth, and the
// bytes of the replicated codebook copies (+ scale table).
template <int F> struct Fm;
template <> struct Fm<kFmtLit> {
  static constexpr int kSb = 48, kSbPerBox = 4, kBoxes = 1, kStages = 2;
  static constexpr int kLut = 256 * 8 * 16;               // 256 entries of 16 bytes, 8 copies
};
template <> struct Fm<kFmtK16> {
  static constexpr int kSb = 80, kSbPerBox = 2, kBoxes = 1, kStages = 2;
  static constexpr int kLut = 2 * 256 * 16 * 8 + 256 * 16 * 2;   // two sub-tables of 8-byte entries, 16 copies; bf16 scales
};
template <> struct Fm<kFmtFp8> {
  static constexpr int kSb = 128, kSbPerBox = 1, kBoxes = 2, kStages = 2;
  static constexpr int kLut = 4 * 256 * 32 * 2;           // four sub-tables of 2-byte entries, 32 copies
};
template <> struct Fm<kFmtF8L> {
  static constexpr int kSb = 64, kSbPerBox = 3, kBoxes = 1, kStages = 2;
  static constexpr int kLut = 2 * 256 * 32 * 4;           // two sub-tables of 4-byte entries, 32 copies
};
template <int F> struct Geo {
  static constexpr int kPitch = Fm<F>::kSbPerBox * Fm<F>::kSb + 16;   // an odd number of 16-byte units
  static constexpr int kBoxBytes = kBM * kPitch;
  static constexpr int kStageBytes = Fm<F>::kBoxes * kBoxBytes;
  static constexpr int kSbPerStage = Fm<F>::kBoxes * Fm<F>::kSbPerBox;
  static constexpr int kFixed = 1024 + Fm<F>::kStages * kStageBytes + Fm<F>::kLut + 512;
  static_assert((kPitch / 16) % 2 == 1 && kPitch <= 256, "row pitch");
};

struct UmmaParams {
  int64_t N, K;
  int M, Mpad;
  int n_sb;                 // superblocks per weight row
  int stages_per_slice;     // raw stages (4 superblocks each) per K slice
  int slices;
  int x_stages;             // activation stages (half a superblock of K each)
  int n_iss;                // MMA issuers = accumulators: 4 (up to 64 activation rows) or 2
  const void* codebook;     // flat codebook block (bf16 for the fp4 grid, E4M3 bytes for the fp8 grid)
  const float* compose;     // two-tier scale table [256, 16] (fp4 k = 16)
  const float* row_scale;   // per weight row (fp8 grid)
  int64_t rows_total;       // rows of the matrix (or of the whole expert stack)
  float global_scale;
  uint16_t* y;              // [M, N] bf16 (one slice)
  float* partial;           // [slices, M, N] fp32 (several slices)
  uint32_t idesc;            // with N = Mpad (dense); grouped mode sets N per pass
  int* status;
  // grouped mode (routed experts): x rows are sorted by expert, expert e owns rows [seg[e], seg[e+1])
  const int32_t* seg;        // [E+1]
  const int32_t* row_map;    // [P] output row of a sorted row, or null = identity
  int tiles_n;               // 128-row tiles per expert
  int n_tiles;               // tiles of the launch (dense: row tiles; grouped: experts x tiles_n)
  uint16_t* y_peer[GB_PEER_MAX];   // optional: output row r lives in y_peer[r / rows_per_rank]
  int64_t rows_per_rank;     // 0 = all rows in y
};

constexpr int kGroupRows = 64;                            // activation rows per pass in grouped mode

GB_DEVINL void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(gb_smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(gb_smem_u32(bar))
      : "memory");
}

// K-major tile of 128-byte rows with the 128-byte swizzle: 8-row groups 1024 bytes apart.
GB_DEVINL uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// D[tmem] (+)= A[tmem] . B[smem]: A holds 128 rows (lanes) x 16 bf16 of K in 8 columns.
GB_DEVINL void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}

GB_DEVINL void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(gb_smem_u32(bar)) : "memory");
}

GB_DEVINL void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]));
}

// A bounded wait that remembers a timeout for the rest of the CTA: later waits return at once.
GB_DEVINL void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (*abort_flag) return;
  if (!gb_mbar_wait(bar, parity)) {
    *abort_flag = 1;
    atomicExch(status, code);
  }
}

GB_DEVINL uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// bf16 pair x fp32 scale, each product rounded to bf16 once (the decode contract's arithmetic when
// the scale is not exact in bf16).
GB_DEVINL uint32_t mul_pair_f32(uint32_t pair, float s) {
  return gb_pack_bf16x2(__uint_as_float(pair << 16) * s, __uint_as_float(pair & 0xFFFF0000u) * s);
}

// The same for the waits on the critical path of every unit: the abort flag is looked at only when
// the barrier is not ready at once.
GB_DEVINL void wait_fast(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(gb_smem_u32(bar)), "r"(parity) : "memory");
  if (done) return;
  wait_or_abort(bar, parity, abort_flag, status, code);
}

// Literal format: four codewords (the bytes of `codes`) of one weight row -> 16 bf16 pairs; `sc2`
// holds the two group scale bytes they share in its low half (low byte: codewords 0 and 1).  A scale
// byte moved into bf16's fields is 2^-120 times its value; the codebook copies carry the 2^120.
// `lut` is the lane's copy of entry 0 as a shared-memory address; entries are 128 bytes apart.
GB_DEVINL void lit_decode4(uint32_t lut, uint32_t codes, uint32_t sc2, uint32_t (&v)[16]) {
  // both scale bytes at once: byte -> (byte & 0x7f) << 4 | (byte & 0x80) << 8 in each half
  const uint32_t x = __byte_perm(sc2, 0u, 0x4140) << 4;                      // [b1 << 4 | b0 << 4] in the halves
  const uint32_t y = (x & 0x07F007F0u) | ((x << 4) & 0x80008000u);
  const uint32_t s2[2] = {__byte_perm(y, y, 0x1010), __byte_perm(y, y, 0x3232)};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    // entry offset = code * 128, straight from the byte's place in the word
    const uint32_t off = (c == 0 ? codes << 7 : codes >> (8 * c - 7)) & 0x7F80u;
    uint4 e;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(e.x), "=r"(e.y), "=r"(e.z), "=r"(e.w) : "r"(lut + off));
    v[c * 4 + 0] = mul_bf16x2(e.x, s2[c >> 1]);
    v[c * 4 + 1] = mul_bf16x2(e.y, s2[c >> 1]);
    v[c * 4 + 2] = mul_bf16x2(e.z, s2[c >> 1]);
    v[c * 4 + 3] = mul_bf16x2(e.w, s2[c >> 1]);
  }
}

// Two-tier product format, k = 16: two index words (four codewords: low byte = first sub-table,
// high byte = second) and the two group scales they use, as bf16 bits (exact) or as fp32.  `lut0` /
// `lut1` are the lane's copies of entry 0 of the two sub-tables (shared-memory addresses, entries
// 128 bytes apart).
template <bool kExact>
GB_DEVINL void k16_decode4(uint32_t lut0, uint32_t lut1, uint32_t wa, uint32_t wb, uint32_t sa, uint32_t sb,
                           float fa, float fb, uint32_t (&v)[16]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t w = c < 2 ? wa : wb;
    const uint32_t off0 = ((c & 1) ? w >> 9 : w << 7) & 0x7F80u, off1 = ((c & 1) ? w >> 17 : w >> 1) & 0x7F80u;
    uint2 e0, e1;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e0.x), "=r"(e0.y) : "r"(lut0 + off0));
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e1.x), "=r"(e1.y) : "r"(lut1 + off1));
    if (kExact) {
      const uint32_t s1 = c < 2 ? sa : sb, s2 = __byte_perm(s1, s1, 0x1010);
      v[c * 4 + 0] = mul_bf16x2(e0.x, s2);
      v[c * 4 + 1] = mul_bf16x2(e0.y, s2);
      v[c * 4 + 2] = mul_bf16x2(e1.x, s2);
      v[c * 4 + 3] = mul_bf16x2(e1.y, s2);
    } else {
      const float f = c < 2 ? fa : fb;
      v[c * 4 + 0] = mul_pair_f32(e0.x, f);
      v[c * 4 + 1] = mul_pair_f32(e0.y, f);
      v[c * 4 + 2] = mul_pair_f32(e1.x, f);
      v[c * 4 + 3] = mul_pair_f32(e1.y, f);
    }
  }
}

// fp8 product format, k = 32: four codewords of four sub-indices; every sub-table entry is two E4M3
// values; weight = bf16(value * row scale), the product taken in fp32.  `lut` is the lane's copy of
// entry 0 of the first sub-table (entries 64 bytes apart, sub-tables 16 KiB apart).
GB_DEVINL void fp8_decode4(uint32_t lut, uint4 cw, float rs, uint32_t (&v)[16]) {
  const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t off = (j == 0 ? w4[c] << 6 : w4[c] >> (8 * j - 6)) & 0x3FC0u;
      uint16_t e;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(e) : "r"(lut + (uint32_t)(j * 16384) + off));
      uint32_t h2;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(e));
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
      v[c * 4 + j] = gb_pack_bf16x2(f.x * rs, f.y * rs);
    }
  }
}

// fp8 product format, k = 16: two index words (four codewords: low byte = first sub-table, high byte
// = second); every sub-table entry is four E4M3 values (entries 128 bytes apart, the second
// sub-table 32 KiB after the first).
GB_DEVINL void f8l_decode4(uint32_t lut, uint32_t wa, uint32_t wb, float rs, uint32_t (&v)[16]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t w = c < 2 ? wa : wb;
    const uint32_t off0 = ((c & 1) ? w >> 9 : w << 7) & 0x7F80u, off1 = ((c & 1) ? w >> 17 : w >> 1) & 0x7F80u;
    uint32_t e[2];
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e[0]) : "r"(lut + off0));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e[1]) : "r"(lut + 32768u + off1));
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      uint32_t lo, hi;
      asm("{\n.reg .b16 a, b;\nmov.b32 {a, b}, %2;\ncvt.rn.f16x2.e4m3x2 %0, a;\ncvt.rn.f16x2.e4m3x2 %1, b;\n}\n"
          : "=r"(lo), "=r"(hi) : "r"(e[t]));
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&lo));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
      v[c * 4 + 2 * t] = gb_pack_bf16x2(f0.x * rs, f0.y * rs);
      v[c * 4 + 2 * t + 1] = gb_pack_bf16x2(f1.x * rs, f1.y * rs);
    }
  }
}

template <bool kGrouped, int F>
__global__ void __launch_bounds__(kUmmaThreads, 1)
umma_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const UmmaParams p) {
  using G = Geo<F>;
  constexpr int kSb = Fm<F>::kSb, kRawStages = Fm<F>::kStages, kSbPerStage = G::kSbPerStage;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int slab_bytes = p.Mpad * 128;                     // one 64-wide K slab of the activations
  const int x_stage_bytes = 2 * slab_bytes;                // half a superblock of K
  uint8_t* xs = smem;                                      // x_stages x (two slabs)
  uint8_t* raw = xs + (size_t)p.x_stages * x_stage_bytes;  // kRawStages x packed rows
  uint8_t* cb_s = raw + kRawStages * G::kStageBytes;       // codebook copies (+ scale table)
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(cb_s + Fm<F>::kLut);
  uint64_t* raw_empty = raw_full + kMaxRawStages;
  uint64_t* full = raw_empty + kMaxRawStages;              // per unit slot: activations landed + operand decoded
  uint64_t* done = full + kMaxXStages;                     // per unit slot: the unit's MMAs have completed
  uint64_t* acc_full = done + kMaxXStages;
  uint64_t* acc_empty = acc_full + 1;                      // grouped mode: the accumulators have been read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* inexact = const_cast<int*>(abort_flag) + 1;         // k = 16: some scale of the table is not exact in bf16

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_raw = (p.n_sb + kSbPerStage - 1) / kSbPerStage;
  const int r_begin = blockIdx.y * p.stages_per_slice;
  const int r_end = min(n_raw, r_begin + p.stages_per_slice);
  const int sb_slice = min(p.n_sb, r_end * kSbPerStage) - r_begin * kSbPerStage;   // superblocks of this K slice
  const int units = 2 * sb_slice;                          // half superblocks per pass
  const uint32_t xs_mask = (uint32_t)p.x_stages - 1u;      // 4 or 8 unit slots
  const int xs_log = p.x_stages == 8 ? 3 : 2;

  gb_pdl_launch_dependents();
  // A CTA walks the 128-row tiles blockIdx.x, blockIdx.x + gridDim.x, ... (codebook copies, tensor
  // memory and barriers are set up once; the rings run on across tiles).  Dense: one pass over rows
  // [0, M) of x per tile.  Grouped: tile = (expert, 128 rows of it), the expert's rows of the sorted
  // x in passes of 64 (the weights are decoded again per pass), nothing to do for an expert
  // without rows.
  if (kGrouped) gb_pdl_wait();                             // the segment offsets come from the routing launch
  const int pass_rows = kGrouped ? kGroupRows : p.Mpad;
  struct Tile { int n0, w_row0, seg_lo, cnt, n_pass; };
  auto tile_at = [&](int t) {
    Tile T;
    T.n0 = t * kBM; T.w_row0 = T.n0; T.seg_lo = 0; T.cnt = p.M;
    if (kGrouped) {
      const int e = t / p.tiles_n;
      T.n0 = (t - e * p.tiles_n) * kBM;
      T.w_row0 = e * (int)p.N + T.n0;
      T.seg_lo = p.seg[e];
      T.cnt = p.seg[e + 1] - T.seg_lo;
    }
    T.n_pass = T.cnt > 0 ? (T.cnt + pass_rows - 1) / pass_rows : 0;
    return T;
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      gb_mbar_init(&raw_full[s], 1);
      gb_mbar_init(&raw_empty[s], kDecWarps);
    }
    for (int s = 0; s < kMaxXStages; ++s) {
      gb_mbar_init(&full[s], 1 + 4);                       // the activation bytes + the four warps of the unit's warpgroup
      gb_mbar_init(&done[s], 1);
    }
    gb_mbar_init(acc_full, (uint32_t)p.n_iss);
    gb_mbar_init(acc_empty, kDecWarps);
    *abort_flag = 0;
    *inexact = 0;
    gb_fence_barrier_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(gb_smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // From here the warps go their own ways: the packed weights do not depend on the launch ahead, so
  // their loads start at once; the decoders build the codebook copies meanwhile; everything that
  // reads x or writes y first waits for the launch ahead.
  //
  // A UNIT is half a superblock of K (128 weights per row).  Unit u of a pass uses operand buffer
  // u mod 4, is decoded by warpgroup u mod 4 and issued by that buffer's issuer; its barriers sit in
  // slot u mod x_stages (4 or 8).  The next completion of done[slot] after unit u is unit u + 4 or
  // u + 8, which the same warpgroup decodes after it has waited for u: no barrier can run ahead of
  // a waiter.

  if (warp == 0) {
    // ------------------------- packed weight rows -------------------------
    if (lane == 0) {
      int it = 0;
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
      const Tile T = tile_at(t);
      for (int pass = 0; pass < T.n_pass; ++pass)
      for (int r = r_begin; r < r_end; ++r, ++it) {
        const int rs = it % kRawStages;
        wait_or_abort(&raw_empty[rs], ((it / kRawStages) & 1) ^ 1, abort_flag, p.status, 21);
        gb_mbar_expect_tx(&raw_full[rs], G::kStageBytes);
#pragma unroll
        for (int bx = 0; bx < Fm<F>::kBoxes; ++bx)
          tma_load_2d(raw + (size_t)rs * G::kStageBytes + bx * G::kBoxBytes, &map_w,
                      (r * kSbPerStage + bx * Fm<F>::kSbPerBox) * kSb, T.w_row0, &raw_full[rs]);
      }
      }
    }
  } else if (warp == 1) {
    // ------------------------- activation slabs ---------------------------
    if (lane == 0) {
      gb_pdl_wait();                                         // x may come from the launch ahead
      const int k_base = r_begin * kSbPerStage * 256;
      int g = 0;                                             // units since the start, over all tiles and passes
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
      const Tile T = tile_at(t);
      for (int pass = 0; pass < T.n_pass; ++pass)
      for (int u = 0; u < units; ++u, ++g) {
        const int s = g & xs_mask;
        wait_or_abort(&done[s], ((uint32_t)(g >> xs_log) & 1u) ^ 1u, abort_flag, p.status, 22);
        gb_mbar_expect_tx(&full[s], (uint32_t)x_stage_bytes);
        uint8_t* dst = xs + (size_t)s * x_stage_bytes;
        const int k0 = k_base + u * 128;
        tma_load_2d(dst, &map_x, k0, T.seg_lo + pass * pass_rows, &full[s]);
        tma_load_2d(dst + slab_bytes, &map_x, k0 + 64, T.seg_lo + pass * pass_rows, &full[s]);
      }
      }
    }
  } else if (warp < kCtlWarps) {
    // ------------------------- MMA issuers ---------------------------------
    // Issuer i takes the units of operand buffer i (four issuers) or of buffers 2i and 2i + 1 (two
    // issuers, when the activation rows leave room for two accumulators only) into its own
    // accumulator; the read-out adds the accumulators in their fixed order.
    const int i = warp - 2;
    if (lane == 0 && i < p.n_iss) {
      const uint32_t acc = tmem_base + (uint32_t)i * (kACol0 / (uint32_t)p.n_iss);
      const uint32_t slab16 = (uint32_t)slab_bytes >> 4;
      const uint64_t desc0 = smem_desc_sw128(gb_smem_u32(xs));
      int g0 = 0, item = 0;                                  // units / (tile, pass) items since the start
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
      const Tile T = tile_at(t);
      for (int pass = 0; pass < T.n_pass; ++pass, g0 += units, ++item) {
        // grouped mode: N = this pass's rows rounded up to 16.  The item before must have been read out.
        uint32_t idesc = p.idesc;
        if (kGrouped) {
          const int rows = min(pass_rows, T.cnt - pass * pass_rows);
          idesc = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)(((rows + 15) / 16 * 16) >> 3) << 17);
        }
        if (item > 0) {
          wait_or_abort(acc_empty, (item - 1) & 1, abort_flag, p.status, 28);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        bool first = true;
        for (int u = 0; u < units; ++u) {
          if ((p.n_iss == 4 ? (u & 3) : ((u >> 1) & 1)) != i) continue;
          const int g = g0 + u, s = g & xs_mask, ab = u & 3;
          wait_fast(&full[s], (uint32_t)(g >> xs_log) & 1u, abort_flag, p.status, 23);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_tmem = tmem_base + kACol0 + (uint32_t)(ab * kABufCols);
          const uint64_t db = desc0 + (uint64_t)((uint32_t)(s * x_stage_bytes) >> 4);
          {
            if (first) {
#pragma unroll
              for (int k = 0; k < 8; ++k)                    // 16 weights of K per instruction
                umma_bf16_ts(acc, a_tmem + (uint32_t)(k * 8), db + (uint64_t)((k >> 2) * slab16 + 2 * (k & 3)), idesc, k > 0);
              first = false;
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k)
                umma_bf16_ts(acc, a_tmem + (uint32_t)(k * 8), db + (uint64_t)((k >> 2) * slab16 + 2 * (k & 3)), idesc, true);
            }
          }
          umma_commit(&done[s]);
        }
        umma_commit(acc_full);
      }
      }
    }
  } else {
    // ------------------------- decoders -------------------------------------
    const int d = threadIdx.x - 32 * kCtlWarps;              // 0 .. 511
    const int de = d & 255, dh = d >> 8;                     // entry, which half of the copies / which table
    if constexpr (F == kFmtLit) {
      // the codebook, eight copies side by side (copy j of an entry sits in the j-th 16-byte bank
      // group), pre-multiplied by 2^120 (exact for the fp4 grid's values)
      const uint4 e = __ldg(reinterpret_cast<const uint4*>(p.codebook) + de);
      const uint32_t two120 = 0x7B807B80u;
      const uint4 w = make_uint4(mul_bf16x2(e.x, two120), mul_bf16x2(e.y, two120), mul_bf16x2(e.z, two120),
                                 mul_bf16x2(e.w, two120));
#pragma unroll
      for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(cb_s)[de * 8 + dh * 4 + j] = w;
    } else if constexpr (F == kFmtK16) {
      // two sub-tables of 256 entries x four bf16, 16 copies each (8-byte loads go 16 lanes at a time);
      // the scale table as bf16, with a note when a value does not survive the conversion
      const uint2 e = __ldg(reinterpret_cast<const uint2*>(p.codebook) + dh * 256 + de);
      uint2* l = reinterpret_cast<uint2*>(cb_s) + dh * 256 * 16;
#pragma unroll
      for (int j = 0; j < 16; ++j) l[de * 16 + j] = e;
      uint16_t* comp_s = reinterpret_cast<uint16_t*>(cb_s + 2 * 256 * 16 * 8);
      bool bad = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = __ldg(p.compose + d * 8 + j);
        const uint32_t b = gb_f32_to_bf16_bits(f);
        bad |= gb_bf16_bits_to_f32(b) != f;
        comp_s[d * 8 + j] = (uint16_t)b;
      }
      if (bad) atomicOr(inexact, 1);
    } else if constexpr (F == kFmtF8L) {
      // two sub-tables of 256 entries x four E4M3 bytes, 32 copies each (one per lane)
      const uint32_t e = __ldg(reinterpret_cast<const uint32_t*>(p.codebook) + dh * 256 + de);
      uint4* l = reinterpret_cast<uint4*>(cb_s) + (dh * 256 + de) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) l[j] = make_uint4(e, e, e, e);
    } else {
      // four sub-tables of 256 entries x two E4M3 bytes, 32 copies each (one per lane)
      const uint16_t* cb = reinterpret_cast<const uint16_t*>(p.codebook);
      uint32_t* l = reinterpret_cast<uint32_t*>(cb_s);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int ent = (dh * 2 + t) * 256 + de;
        const uint32_t e2 = (uint32_t)__ldg(cb + ent) * 0x10001u;
#pragma unroll
        for (int j = 0; j < 16; ++j) l[ent * 16 + j] = e2;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecWarps) : "memory");
    gb_pdl_wait();                                           // y may still be read by the launch ahead
    const int quarter = warp & 3;                            // the tensor-memory lanes this warp may touch
    const int wg = (warp - kCtlWarps) >> 2;                  // warpgroup = operand buffer: units wg, wg + 4, ...
    const int h = wg & 1;                                    // its half of a superblock ...
    const int sb_par = wg >> 1;                              // ... of the even or the odd superblocks
    const int row = quarter * 32 + lane;                     // weight row of the tile = tensor-memory lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t col = lane_base + kACol0 + (uint32_t)(wg * kABufCols);
    const bool exact = *inexact == 0;
    int it = 0, g_sb = 0, item = 0;                          // raw stages, superblocks, (tile, pass) items so far
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x) {
    const Tile T = tile_at(t);
    float rs = 0.0f;                                         // fp8 grid: this row's scale
    if constexpr (F == kFmtFp8 || F == kFmtF8L) {
      if (T.n_pass > 0 && (int64_t)T.w_row0 + row < p.rows_total) rs = __ldg(p.row_scale + T.w_row0 + row);
    }
    for (int pass = 0; pass < T.n_pass; ++pass, ++item) {
    for (int r = r_begin; r < r_end; ++r, ++it) {
      const int rs_i = it % kRawStages;
      wait_or_abort(&raw_full[rs_i], (it / kRawStages) & 1, abort_flag, p.status, 24);
      const uint8_t* stage = raw + (size_t)rs_i * G::kStageBytes;
      const int sb_here = min(kSbPerStage, p.n_sb - r * kSbPerStage);
      for (int sbi = 0; sbi < sb_here; ++sbi, ++g_sb) {
        // superblock number inside the pass decides the warpgroup (the passes of a grouped launch
        // all start at unit 0)
        const int sb_in_pass = (r - r_begin) * kSbPerStage + sbi;
        if ((sb_in_pass & 1) != sb_par) continue;
        const int g = 2 * g_sb + h, s = g & xs_mask;         // unit since the start, its barrier slot
        const uint4* rp = reinterpret_cast<const uint4*>(stage + (sbi / Fm<F>::kSbPerBox) * G::kBoxBytes + row * G::kPitch +
                                                         (sbi % Fm<F>::kSbPerBox) * kSb);
        uint32_t v0[16], v1[16];
        // ---- first eight codewords into registers, then wait for the operand buffer ----
        if constexpr (F == kFmtLit) {
          const uint32_t lut = gb_smem_u32(cb_s) + (uint32_t)(lane & 7) * 16u;
          const uint4 cw = rp[h];
          const uint2 sc = reinterpret_cast<const uint2*>(rp + 2)[h];
          lit_decode4(lut, cw.x, sc.x & 0xFFFFu, v0);
          lit_decode4(lut, cw.y, sc.x >> 16, v1);
          if (sb_in_pass >= 2) wait_fast(&done[(g - 4) & xs_mask], (uint32_t)((g - 4) >> xs_log) & 1u, abort_flag, p.status, 25);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          tmem_st16(col, v0);
          tmem_st16(col + 16u, v1);
          lit_decode4(lut, cw.z, sc.y & 0xFFFFu, v0);
          lit_decode4(lut, cw.w, sc.y >> 16, v1);
          tmem_st16(col + 32u, v0);
          tmem_st16(col + 48u, v1);
        } else if constexpr (F == kFmtK16) {
          const uint32_t lut0 = gb_smem_u32(cb_s) + (uint32_t)(lane & 15) * 8u, lut1 = lut0 + 256u * 16u * 8u;
          const uint16_t* comp_s = reinterpret_cast<const uint16_t*>(cb_s + 2 * 256 * 16 * 8);
          const uint4 ia = rp[2 * h], ib = rp[2 * h + 1], q4 = rp[4];    // eight index words: sixteen codewords
          const uint16_t* crow = comp_s + (q4.x & 0xFFu) * 16;
          const float* frow = p.compose + (q4.x & 0xFFu) * 16;
          const uint32_t nib = h ? __funnelshift_r(q4.y, q4.z, 8) : __funnelshift_r(q4.x, q4.y, 8);   // eight group codes
          auto four = [&](uint32_t wa, uint32_t wb, uint32_t n2, uint32_t (&v)[16]) {
            const uint32_t na = n2 & 0xFu, nb = (n2 >> 4) & 0xFu;
            if (exact) k16_decode4<true>(lut0, lut1, wa, wb, crow[na], crow[nb], 0.0f, 0.0f, v);
            else k16_decode4<false>(lut0, lut1, wa, wb, 0u, 0u, __ldg(frow + na), __ldg(frow + nb), v);
          };
          four(ia.x, ia.y, nib, v0);
          four(ia.z, ia.w, nib >> 8, v1);
          if (sb_in_pass >= 2) wait_fast(&done[(g - 4) & xs_mask], (uint32_t)((g - 4) >> xs_log) & 1u, abort_flag, p.status, 25);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          tmem_st16(col, v0);
          tmem_st16(col + 16u, v1);
          four(ib.x, ib.y, nib >> 16, v0);
          four(ib.z, ib.w, nib >> 24, v1);
          tmem_st16(col + 32u, v0);
          tmem_st16(col + 48u, v1);
        } else if constexpr (F == kFmtF8L) {
          const uint32_t lut = gb_smem_u32(cb_s) + (uint32_t)lane * 4u;
          const uint4 ia = rp[2 * h], ib = rp[2 * h + 1];    // eight index words: sixteen codewords
          f8l_decode4(lut, ia.x, ia.y, rs, v0);
          f8l_decode4(lut, ia.z, ia.w, rs, v1);
          if (sb_in_pass >= 2) wait_fast(&done[(g - 4) & xs_mask], (uint32_t)((g - 4) >> xs_log) & 1u, abort_flag, p.status, 25);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          tmem_st16(col, v0);
          tmem_st16(col + 16u, v1);
          f8l_decode4(lut, ib.x, ib.y, rs, v0);
          f8l_decode4(lut, ib.z, ib.w, rs, v1);
          tmem_st16(col + 32u, v0);
          tmem_st16(col + 48u, v1);
        } else {
          const uint32_t lut = gb_smem_u32(cb_s) + (uint32_t)lane * 2u;
          fp8_decode4(lut, rp[4 * h], rs, v0);
          fp8_decode4(lut, rp[4 * h + 1], rs, v1);
          if (sb_in_pass >= 2) wait_fast(&done[(g - 4) & xs_mask], (uint32_t)((g - 4) >> xs_log) & 1u, abort_flag, p.status, 25);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          tmem_st16(col, v0);
          tmem_st16(col + 16u, v1);
          fp8_decode4(lut, rp[4 * h + 2], rs, v0);
          fp8_decode4(lut, rp[4 * h + 3], rs, v1);
          tmem_st16(col + 32u, v0);
          tmem_st16(col + 48u, v1);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) gb_mbar_arrive(&full[s]);
      }
      __syncwarp();
      if (lane == 0) gb_mbar_arrive(&raw_empty[rs_i]);
    }

    // ------------------------- read-out ------------------------------------
    wait_or_abort(acc_full, item & 1, abort_flag, p.status, 26);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int col_part = (warp - kCtlWarps) >> 2;            // column chunks: every fourth
    // issuers that had no unit in this slice leave their accumulator untouched
    const int n_accs = min(p.n_iss, p.n_iss == 4 ? units : sb_slice);
    const uint32_t acc_stride = kACol0 / (uint32_t)p.n_iss;
    const int64_t out_col = (int64_t)T.n0 + row;
    const bool ok = *abort_flag == 0;
    const int rows = min(pass_rows, T.cnt - pass * pass_rows);
    for (int c = col_part; c < (rows + 7) / 8; c += kDecWarps / 4) {
      uint32_t v[8];
      const uint32_t taddr = lane_base + (uint32_t)(c * 8);
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      for (int a = 1; a < n_accs; ++a) {                     // the other issuers' accumulators, in their fixed order
        uint32_t t[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3]), "=r"(t[4]), "=r"(t[5]), "=r"(t[6]), "=r"(t[7])
                     : "r"(taddr + (uint32_t)a * acc_stride));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(t[i]));
      }
      if (ok && out_col < p.N) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = c * 8 + i;
          if (m < rows) {
            if (kGrouped) {
              const int jrow = T.seg_lo + pass * pass_rows + m;        // sorted position of the row
              int64_t orow = p.row_map ? p.row_map[jrow] : jrow;
              uint16_t* ybase = p.y;
              if (p.rows_per_rank > 0) {                     // the row's home rank keeps it (peer store)
                const int64_t home = orow / p.rows_per_rank;
                ybase = p.y_peer[home];
                orow -= home * p.rows_per_rank;
              }
              ybase[orow * p.N + out_col] = (uint16_t)gb_f32_to_bf16_bits(__uint_as_float(v[i]) * p.global_scale);
            } else if (p.slices > 1) {
              p.partial[((int64_t)blockIdx.y * p.M + m) * p.N + out_col] = __uint_as_float(v[i]);
            } else {
              p.y[(int64_t)m * p.N + out_col] = (uint16_t)gb_f32_to_bf16_bits(__uint_as_float(v[i]) * p.global_scale);
            }
          }
        }
      }
    }
    // hand the accumulators back for the next item (pass or tile)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) gb_mbar_arrive(acc_empty);
    }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// y[m][n] = bf16(global_scale * sum over the K slices), in slice order.
__global__ void __launch_bounds__(256)
umma_finalize_kernel(const float* __restrict__ partial, int slices, int64_t MN, float global_scale,
                     uint16_t* __restrict__ y) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= MN) return;
  float acc = 0.0f;
  for (int s = 0; s < slices; ++s) acc += partial[(int64_t)s * MN + i];
  y[i] = (uint16_t)gb_f32_to_bf16_bits(acc * global_scale);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct FmtInfo {
  int sb_bytes, sb_per_stage, pitch, fixed_smem;
};

FmtInfo fmt_info(int F) {
  switch (F) {
    case kFmtLit: return {Fm<kFmtLit>::kSb, Geo<kFmtLit>::kSbPerStage, Geo<kFmtLit>::kPitch, Geo<kFmtLit>::kFixed};
    case kFmtK16: return {Fm<kFmtK16>::kSb, Geo<kFmtK16>::kSbPerStage, Geo<kFmtK16>::kPitch, Geo<kFmtK16>::kFixed};
    case kFmtF8L: return {Fm<kFmtF8L>::kSb, Geo<kFmtF8L>::kSbPerStage, Geo<kFmtF8L>::kPitch, Geo<kFmtF8L>::kFixed};
    default: return {Fm<kFmtFp8>::kSb, Geo<kFmtFp8>::kSbPerStage, Geo<kFmtFp8>::kPitch, Geo<kFmtFp8>::kFixed};
  }
}

// Activation stages: eight where the format's rings and tables leave room, else four, else none (0:
// the kernel does not take the shape).  Only these two depths are safe: a decoder learns that its
// operand buffer is free from the activation-stage barrier of the unit four back, and that barrier
// must not complete again before the decoder has looked (with four stages its next completion is
// the decoder's own unit, with eight a later unit of the same warpgroup).
int umma_x_stages(int F, int Mpad) {
  const int n = (kSmemCap - fmt_info(F).fixed_smem) / (2 * Mpad * 128);
  return n >= 8 ? 8 : n >= 4 ? 4 : 0;
}

int umma_smem_bytes(int F, int Mpad) { return fmt_info(F).fixed_smem + umma_x_stages(F, Mpad) * (2 * Mpad * 128); }

// K slices: enough CTAs for the SMs when the layer has few 128-row tiles.
void umma_plan(int F, int64_t N, int n_sb, int sms, int* slices, int* stages_per_slice) {
  const int per_stage = fmt_info(F).sb_per_stage;
  const int tiles = (int)((N + kBM - 1) / kBM);
  const int n_raw = (n_sb + per_stage - 1) / per_stage;
  int want = sms / tiles;
  if (want < 1) want = 1;
  if (want > n_raw) want = n_raw;
  *stages_per_slice = (n_raw + want - 1) / want;
  *slices = (n_raw + *stages_per_slice - 1) / *stages_per_slice;
}

// Which decoder serves the weight, or -1.  The two-tier format is taken with its superblocks padded
// to 80 bytes only (type_size 80): 73-byte superblocks cannot be fetched by tiled TMA.
int umma_format(const gb_weight* w) {
  const gb_format& f = w->fmt;
  if (w->cb_row_offset != nullptr || (w->row_stride % 16) != 0 || ((uintptr_t)w->qw & 15u) != 0 ||
      ((uintptr_t)w->codebook & 15u) != 0)
    return -1;
  if (f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
      f.type_size == Fm<kFmtLit>::kSb)
    return kFmtLit;
  if (f.grid == GB_GRID_FP4 && f.mode == GB_MODE_PRODUCT && f.n_sub == 2 && f.k_bits == 16 &&
      f.scale_coding == GB_SCALE_V2 && f.type_size == Fm<kFmtK16>::kSb && w->compose != nullptr)
    return kFmtK16;
  if (f.grid == GB_GRID_FP8 && f.mode == GB_MODE_PRODUCT && f.n_sub == 4 && f.k_bits == 32 &&
      f.type_size == Fm<kFmtFp8>::kSb && w->weight_scale != nullptr)
    return kFmtFp8;
  if (f.grid == GB_GRID_FP8 && f.mode == GB_MODE_PRODUCT && f.n_sub == 2 && f.k_bits == 16 &&
      f.type_size == Fm<kFmtF8L>::kSb && w->weight_scale != nullptr)
    return kFmtF8L;
  return -1;
}

bool umma_applies(const gb_weight* w, int64_t M) {
  const int F = umma_format(w);
  return F >= 0 && M >= 1 && M <= kMaxRows && w->K >= 1024 && w->rows >= kBM && umma_x_stages(F, (int)((M + 15) / 16 * 16)) >= 4;
}

template <bool kGrouped>
cudaError_t launch_umma(int F, dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap& map_w,
                        const CUtensorMap& map_x, const UmmaParams& p) {
  switch (F) {
    case kFmtLit: return gb_launch(umma_decode_kernel<kGrouped, kFmtLit>, grid, dim3(kUmmaThreads), smem, stream, map_w, map_x, p);
    case kFmtK16: return gb_launch(umma_decode_kernel<kGrouped, kFmtK16>, grid, dim3(kUmmaThreads), smem, stream, map_w, map_x, p);
    case kFmtF8L: return gb_launch(umma_decode_kernel<kGrouped, kFmtF8L>, grid, dim3(kUmmaThreads), smem, stream, map_w, map_x, p);
    default: return gb_launch(umma_decode_kernel<kGrouped, kFmtFp8>, grid, dim3(kUmmaThreads), smem, stream, map_w, map_x, p);
  }
}

void fill_weight_params(UmmaParams& p, const gb_weight* w, int64_t rows_total) {
  p.codebook = w->codebook;
  p.compose = (const float*)w->compose;
  p.row_scale = (const float*)w->weight_scale;
  p.rows_total = rows_total;
  p.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
}

}  // namespace

int gb_prepare_umma() {
#define GB_UMMA_ATTR(G, F, rows)                                                                          \
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)umma_decode_kernel<G, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  kSmemCap))
  GB_UMMA_ATTR(false, kFmtLit, kMaxRows);
  GB_UMMA_ATTR(false, kFmtK16, kMaxRows);
  GB_UMMA_ATTR(false, kFmtFp8, kMaxRows);
  GB_UMMA_ATTR(false, kFmtF8L, kMaxRows);
  GB_UMMA_ATTR(true, kFmtLit, kGroupRows);
  GB_UMMA_ATTR(true, kFmtK16, kGroupRows);
  GB_UMMA_ATTR(true, kFmtFp8, kGroupRows);
  GB_UMMA_ATTR(true, kFmtF8L, kGroupRows);
#undef GB_UMMA_ATTR
  return GB_OK;
}

// An upper bound over the formats: the bucketed activations plus one fp32 partial plane per K slice
// (never more slices than SMs per row tile).
int64_t gb_gemv_umma_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M < 1 || M > kMaxRows || K < 1024 || N < kBM) return 0;
  const int64_t xq = (M * K * 2 + 255) & ~255ll;
  int sms = gb_sm_count();
  if (sms <= 0) sms = 148;
  int most = 1;
  for (int F = 0; F < 4; ++F) {
    int slices, per;
    umma_plan(F, N, (int)(K / 256), sms, &slices, &per);
    if (slices > most) most = slices;
  }
  return xq + (most > 1 ? (int64_t)most * M * N * 4 : 0);
}

int gb_gemv_umma(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                 int64_t workspace_bytes, void* stream_) {
  if (!umma_applies(w, M) || ((uintptr_t)x & 15u) != 0) return GB_EUNSUPPORTED;
  const int F = umma_format(w);
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  const int64_t N = w->rows, K = w->K;
  const FmtInfo fi = fmt_info(F);
  UmmaParams p = {};
  p.N = N; p.K = K; p.M = (int)M; p.Mpad = (int)((M + 15) / 16 * 16);
  p.n_sb = (int)(K / 256);
  umma_plan(F, N, p.n_sb, sms, &p.slices, &p.stages_per_slice);
  const int64_t xq_bytes = act == GB_ACT_NONE ? 0 : ((M * K * 2 + 255) & ~255ll);
  const int64_t part_bytes = p.slices > 1 ? (int64_t)p.slices * M * N * 4 : 0;
  if (xq_bytes + part_bytes > 0 && (workspace == nullptr || workspace_bytes < xq_bytes + part_bytes))
    return gb_fail(GB_EWORKSPACE, "workspace of %lld bytes is too small (need %lld)", (long long)workspace_bytes,
                   (long long)(xq_bytes + part_bytes));
  const void* xin = x;
  if (act != GB_ACT_NONE) {
    int rc = act == GB_ACT_FP4_GROUP16 ? gb_fp4_act_qdq(x, workspace, M, K, scale_rule, stream_)
                                       : gb_fp8_act_qdq(x, workspace, M, K, scale_rule, stream_);
    if (rc != GB_OK) return rc;
    xin = workspace;
  }
  CUtensorMap map_w, map_x;
  int rc = gb_tensor_map_bytes_2d(&map_w, w->qw, (uint64_t)p.n_sb * fi.sb_bytes, (uint64_t)N, (uint64_t)w->row_stride,
                                  fi.pitch, kBM);
  if (rc != GB_OK) return rc;
  rc = gb_tensor_map_operand(&map_x, xin, M, K, 2, p.Mpad);
  if (rc != GB_OK) return rc;
  fill_weight_params(p, w, N);
  p.y = (uint16_t*)y;
  p.partial = p.slices > 1 ? (float*)((uint8_t*)workspace + xq_bytes) : nullptr;
  // fp32 accumulate, bf16 x bf16, both K-major, N = activation rows (padded), M = 128 weight rows
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.Mpad >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.x_stages = umma_x_stages(F, p.Mpad);
  p.n_iss = p.Mpad <= 64 ? 4 : 2;
  p.status = gb_status_word();
  // one CTA per SM at most: a CTA walks several row tiles when the layer has more of them
  p.n_tiles = (int)((N + kBM - 1) / kBM);
  const int ctas_x = p.n_tiles * p.slices <= sms ? p.n_tiles : (sms / p.slices > 0 ? sms / p.slices : 1);
  dim3 grid((unsigned)ctas_x, (unsigned)p.slices);
  GB_CUDA_OK(launch_umma<false>(F, grid, (size_t)umma_smem_bytes(F, p.Mpad), (cudaStream_t)stream_, map_w, map_x, p));
  if (p.slices > 1) {
    const int64_t MN = M * N;
    GB_CUDA_OK(gb_launch(umma_finalize_kernel, dim3((unsigned)((MN + 255) / 256)), dim3(256), 0,
                         (cudaStream_t)stream_, (const float*)p.partial, p.slices, MN, p.global_scale,
                         (uint16_t*)y));
  }
  return GB_OK;
}

// Most activation rows the tensor-core decode kernel takes for this weight (0: not its format or
// layout): what the format's rings and tables leave for four activation stages.
int gb_gemv_umma_max_rows(const gb_weight* w) {
  const int F = umma_format(w);
  if (F < 0 || w->K < 1024 || w->rows < kBM) return 0;
  int best = 0;
  for (int m = 16; m <= kMaxRows; m += 16)
    if (umma_x_stages(F, m) >= 4) best = m;
  return best;
}

bool gb_gemv_umma_is_literal(const gb_weight* w) { return umma_format(w) == kFmtLit; }

extern "C" {

int gb_moe_gemv_sorted(const void* x_sorted, const gb_weight* w, int64_t expert_stride, int64_t E,
                       const int32_t* seg_offsets, const int32_t* row_map, int64_t P, void* y,
                       const gb_peer_rows* y_rows, void* stream_) {
  GB_REQUIRE(x_sorted && w && seg_offsets && (y || y_rows), "null pointer argument");
  GB_REQUIRE(E >= 1 && P >= 0, "bad shape E=%lld P=%lld", (long long)E, (long long)P);
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  const int64_t N = w->rows, K = w->K;
  const int F = umma_format(w);
  if (!(F >= 0 && N % kBM == 0 && expert_stride == N * w->row_stride && ((uintptr_t)x_sorted & 15u) == 0 &&
        E * N < (1ll << 31)))
    return gb_fail(GB_EUNSUPPORTED,
                   "the sorted-rows expert kernel takes contiguous stacks of the literal fp4 format, the two-tier k = 16 "
                   "format with 80-byte superblocks or the fp8 product formats k = 32 / k = 16, with N %% 128 == 0 and one codebook");
  if (P == 0) return GB_OK;
  if (gb_sm_count() <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  const FmtInfo fi = fmt_info(F);
  UmmaParams p = {};
  p.N = N; p.K = K; p.M = kGroupRows; p.Mpad = kGroupRows;
  p.n_sb = (int)(K / 256);
  p.slices = 1;
  p.stages_per_slice = (p.n_sb + fi.sb_per_stage - 1) / fi.sb_per_stage;
  CUtensorMap map_w, map_x;
  rc = gb_tensor_map_bytes_2d(&map_w, w->qw, (uint64_t)p.n_sb * fi.sb_bytes, (uint64_t)(E * N), (uint64_t)w->row_stride,
                              fi.pitch, kBM);
  if (rc != GB_OK) return rc;
  rc = gb_tensor_map_operand(&map_x, x_sorted, P, K, 2, kGroupRows);
  if (rc != GB_OK) return rc;
  fill_weight_params(p, w, E * N);
  p.y = (uint16_t*)y;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kGroupRows >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.x_stages = umma_x_stages(F, kGroupRows);
  p.n_iss = 4;
  p.status = gb_status_word();
  p.seg = seg_offsets; p.row_map = row_map;
  p.tiles_n = (int)(N / kBM);
  if (y_rows) {
    GB_REQUIRE(y_rows->rows_per_rank > 0, "per-rank output rows need rows_per_rank > 0");
    const int64_t ranks = (P + y_rows->rows_per_rank - 1) / y_rows->rows_per_rank;
    GB_REQUIRE(ranks <= GB_PEER_MAX, "output rows span %lld ranks", (long long)ranks);
    for (int r = 0; r < (int)ranks; ++r) {
      GB_REQUIRE(y_rows->base[r] != nullptr, "output buffer of rank %d is null", r);
      p.y_peer[r] = (uint16_t*)y_rows->base[r];
    }
    p.rows_per_rank = y_rows->rows_per_rank;
  }
  p.n_tiles = (int)(E * p.tiles_n);
  const int sms = gb_sm_count();
  dim3 grid((unsigned)(p.n_tiles < sms ? p.n_tiles : sms), 1);
  GB_CUDA_OK(launch_umma<true>(F, grid, (size_t)umma_smem_bytes(F, kGroupRows), (cudaStream_t)stream_, map_w, map_x, p));
  return GB_OK;
}

}  // extern "C"
