// Decode-batch linear of the literal format on the tensor cores, without a decoded copy in HBM:
// y[M, N] = x[M, K] . W^T for 2 <= M <= 128 activation rows.
//
// The WEIGHTS are the M side of the MMA: a CTA owns 128 weight rows and a K slice.  One warp
// streams the packed rows (4 superblocks = 192 bytes per row and stage) into shared memory with
// tiled TMA loads, one warp streams the matching 64-wide K slabs of the (bucketed) activations
// with the 128-byte swizzle, eight warps decode: a thread takes one codeword (code byte ->
// 16-byte codebook entry from a shared-memory copy, group scale byte -> bf16 pair by three
// integer operations, four packed bf16 multiplies = bf16(value * scale), the decode contract) and
// stores the eight weights as one 16-byte chunk at its swizzled place of a K-major 128 x 64 bf16
// slab.  One thread issues tcgen05.mma (M = 128 weight rows, N = activation rows padded to 16,
// kind::f16) on the decoded slab and the activation slab; the fp32 accumulator lives in tensor
// memory and never leaves it during the K loop.  The decoders read it out at the end (lane =
// weight row, column = activation row) and store bf16, or fp32 partial sums per K slice that a
// small second kernel adds.
#include "gb_common.cuh"

#include <cuda.h>

namespace {

constexpr int kBM = 128;                                  // weight rows per CTA
constexpr int kRawSb = 4;                                 // superblocks per raw stage
constexpr int kSbBytes = 48;                              // literal superblock: 32 codes + 16 scales
constexpr int kRawRowBytes = kRawSb * kSbBytes;           // 192
constexpr int kRawStageBytes = kBM * kRawRowBytes;        // 24 KiB
constexpr int kRawSbBytes = kBM * kSbBytes;               // one superblock column of a stage: 48-byte rows
constexpr int kRawStages = 3;
constexpr int kSlabStages = 4;
constexpr int kASlabBytes = kBM * 128;                    // 128 rows x 64 bf16
constexpr int kDecWarps = 8;
constexpr int kCtlWarps = 3;                              // raw producer, x producer, MMA issuer
constexpr int kUmmaThreads = 32 * (kCtlWarps + kDecWarps);
constexpr int kMaxRows = 128;                             // activation rows

struct UmmaParams {
  int64_t N, K;
  int M, Mpad;
  int n_sb;                 // superblocks per weight row
  int stages_per_slice;     // raw stages (4 superblocks each) per K slice
  int slices;
  const uint4* codebook;    // 256 entries of eight bf16
  float global_scale;
  uint16_t* y;              // [M, N] bf16 (one slice)
  float* partial;           // [slices, M, N] fp32 (several slices)
  uint32_t idesc;            // with N = Mpad (dense); grouped mode sets N per pass
  uint32_t tmem_cols;
  int* status;
  // grouped mode (routed experts): x rows are sorted by expert, expert e owns rows [seg[e], seg[e+1])
  const int32_t* seg;        // [E+1]
  const int32_t* row_map;    // [P] output row of a sorted row, or null = identity
  int tiles_n;               // 128-row tiles per expert
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

GB_DEVINL void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
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
__global__ void __launch_bounds__(kUmmaThreads, 1)
umma_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int b_bytes = p.Mpad * 128;                        // one activation slab
  const int slab_bytes = kASlabBytes + b_bytes;
  uint8_t* slabs = smem;                                   // kSlabStages x (A slab | x slab)
  uint8_t* raw = slabs + kSlabStages * slab_bytes;         // kRawStages x packed rows
  uint4* cb_s = reinterpret_cast<uint4*>(raw + kRawStages * kRawStageBytes);
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(cb_s + 256);
  uint64_t* raw_empty = raw_full + kRawStages;
  uint64_t* slab_full = raw_empty + kRawStages;
  uint64_t* slab_empty = slab_full + kSlabStages;
  uint64_t* acc_full = slab_empty + kSlabStages;
  uint64_t* acc_empty = acc_full + 1;                      // grouped mode: the accumulator has been read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_raw = (p.n_sb + kRawSb - 1) / kRawSb;
  const int r_begin = blockIdx.y * p.stages_per_slice;
  const int r_end = min(n_raw, r_begin + p.stages_per_slice);

  gb_pdl_launch_dependents();
  // Dense: one pass over rows [0, M) of x.  Grouped: the CTA's expert, its rows of the sorted x in
  // passes of 64 (the weights are decoded again per pass), nothing to do for an expert without rows.
  int n0 = blockIdx.x * kBM, w_row0 = n0, seg_lo = 0, cnt = p.M;
  if (kGrouped) {
    gb_pdl_wait();                                         // the segment offsets come from the routing launch
    const int e = blockIdx.x / p.tiles_n;
    n0 = (blockIdx.x - e * p.tiles_n) * kBM;
    w_row0 = e * (int)p.N + n0;
    seg_lo = p.seg[e];
    cnt = p.seg[e + 1] - seg_lo;
    if (cnt <= 0) return;
  }
  const int pass_rows = kGrouped ? kGroupRows : p.Mpad;
  const int n_pass = (cnt + pass_rows - 1) / pass_rows;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      gb_mbar_init(&raw_full[s], 1);
      gb_mbar_init(&raw_empty[s], kDecWarps);
    }
    for (int s = 0; s < kSlabStages; ++s) {
      gb_mbar_init(&slab_full[s], 1 + kDecWarps);          // the x slab's bytes + every decoder warp
      gb_mbar_init(&slab_empty[s], 1);
    }
    gb_mbar_init(acc_full, 1);
    gb_mbar_init(acc_empty, kDecWarps);
    *abort_flag = 0;
    gb_fence_barrier_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(gb_smem_u32(tmem_slot)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp >= kCtlWarps) {
    // constant of the layer: the codebook
    const int d = threadIdx.x - 32 * kCtlWarps;
    // The group scale is used as the E4M3 byte moved into bf16's fields, i.e. 2^-120 times its
    // value (exact, subnormal codes included); the codebook copy carries the 2^120 (exact for the
    // fp4 grid's values), so the packed multiply still rounds the exact product value * scale once.
    const uint4 e = __ldg(p.codebook + d);
    uint4 w;
    const uint32_t two120 = 0x7B807B80u;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.x) : "r"(e.x), "r"(two120));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.y) : "r"(e.y), "r"(two120));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.z) : "r"(e.z), "r"(two120));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.w) : "r"(e.w), "r"(two120));
    cb_s[d] = w;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  gb_pdl_wait();                                           // x may come from the launch ahead

  if (warp == 0) {
    // ------------------------- packed weight rows -------------------------
    if (lane == 0) {
      for (int pass = 0, it = 0; pass < n_pass; ++pass)
      for (int r = r_begin; r < r_end; ++r, ++it) {
        const int rs = it % kRawStages;
        wait_or_abort(&raw_empty[rs], ((it / kRawStages) & 1) ^ 1, abort_flag, p.status, 21);
        gb_mbar_expect_tx(&raw_full[rs], kRawStageBytes);
        // one box per superblock column: with 48-byte rows in shared memory the four rows a decoder
        // warp reads at a time sit on different banks (192-byte rows would share two)
#pragma unroll
        for (int sbi = 0; sbi < kRawSb; ++sbi)
          tma_load_2d(raw + (size_t)rs * kRawStageBytes + sbi * kRawSbBytes, &map_w,
                      r * kRawRowBytes + sbi * kSbBytes, w_row0, &raw_full[rs]);
      }
    }
  } else if (warp == 1) {
    // ------------------------- activation slabs ---------------------------
    if (lane == 0) {
      int slab = 0;
      for (int pass = 0; pass < n_pass; ++pass)
      for (int r = r_begin; r < r_end; ++r) {
        const int n_here = min(kRawSb, p.n_sb - r * kRawSb) * 4;       // slabs of this raw stage
        for (int q = 0; q < n_here; ++q, ++slab) {
          const int s = slab % kSlabStages;
          wait_or_abort(&slab_empty[s], ((slab / kSlabStages) & 1) ^ 1, abort_flag, p.status, 22);
          gb_mbar_expect_tx(&slab_full[s], (uint32_t)b_bytes);
          tma_load_2d(slabs + (size_t)s * slab_bytes + kASlabBytes, &map_x, r * (kRawSb * 256) + q * 64,
                      seg_lo + pass * pass_rows, &slab_full[s]);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------- MMA issuer ----------------------------------
    if (lane == 0) {
      int slab = 0;
      for (int pass = 0; pass < n_pass; ++pass) {
      // grouped mode: N = this pass's rows rounded up to 16; the previous pass must have been read out
      uint32_t idesc = p.idesc;
      if (kGrouped) {
        const int rows = min(pass_rows, cnt - pass * pass_rows);
        idesc = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)(((rows + 15) / 16 * 16) >> 3) << 17);
        if (pass > 0) {
          wait_or_abort(acc_empty, (pass - 1) & 1, abort_flag, p.status, 28);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
      }
      const int slab0 = slab;
      for (int r = r_begin; r < r_end; ++r) {
        const int n_here = min(kRawSb, p.n_sb - r * kRawSb) * 4;
        for (int q = 0; q < n_here; ++q, ++slab) {
          const int s = slab % kSlabStages;
          wait_or_abort(&slab_full[s], (slab / kSlabStages) & 1, abort_flag, p.status, 23);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = gb_smem_u32(slabs + (size_t)s * slab_bytes);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + kASlabBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)                        // 16 weights of K per instruction
            umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, slab > slab0 || k > 0);
          umma_commit(&slab_empty[s]);
        }
      }
      umma_commit(acc_full);
      }
    }
  } else {
    // ------------------------- decoders -------------------------------------
    const int d = threadIdx.x - 32 * kCtlWarps;
    const int j = d & 7, rsub = d >> 3;                      // codeword of the slab row, row inside a 32-row band
    int slab = 0, it = 0;
    for (int pass = 0; pass < n_pass; ++pass) {
    for (int r = r_begin; r < r_end; ++r, ++it) {
      const int rs = it % kRawStages;
      wait_or_abort(&raw_full[rs], (it / kRawStages) & 1, abort_flag, p.status, 24);
      const uint8_t* stage = raw + (size_t)rs * kRawStageBytes;
      const int sb_here = min(kRawSb, p.n_sb - r * kRawSb);
      for (int sbi = 0; sbi < sb_here; ++sbi) {
        for (int q = 0; q < 4; ++q, ++slab) {
          const int s = slab % kSlabStages;
          wait_or_abort(&slab_empty[s], ((slab / kSlabStages) & 1) ^ 1, abort_flag, p.status, 25);
          uint8_t* a_slab = slabs + (size_t)s * slab_bytes;
          uint32_t code[4], sc[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint8_t* rp = stage + sbi * kRawSbBytes + (i * 32 + rsub) * kSbBytes;
            code[i] = rp[q * 8 + j];
            sc[i] = rp[32 + q * 4 + (j >> 1)];
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = i * 32 + rsub;
            const uint4 e = cb_s[code[i]];
            const uint32_t s2 = (((sc[i] & 0x7Fu) << 4) | ((sc[i] & 0x80u) << 8)) * 0x10001u;
            uint4 w;
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.x) : "r"(e.x), "r"(s2));
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.y) : "r"(e.y), "r"(s2));
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.z) : "r"(e.z), "r"(s2));
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w.w) : "r"(e.w), "r"(s2));
            *reinterpret_cast<uint4*>(a_slab + (row >> 3) * 1024 + (row & 7) * 128 + ((j ^ (row & 7)) << 4)) = w;
          }
          // generic-proxy stores -> visible to the tensor core's async proxy, then one arrival per warp
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) gb_mbar_arrive(&slab_full[s]);
        }
      }
      __syncwarp();
      if (lane == 0) gb_mbar_arrive(&raw_empty[rs]);
    }

    // ------------------------- read-out ------------------------------------
    wait_or_abort(acc_full, pass & 1, abort_flag, p.status, 26);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int quarter = warp & 3;                            // the tensor-memory lanes this warp may read
    const int col_half = (warp - kCtlWarps) >> 2;            // column chunks: even / odd
    const int64_t out_col = (int64_t)n0 + quarter * 32 + lane;
    const bool ok = *abort_flag == 0;
    const int rows = min(pass_rows, cnt - pass * pass_rows);
    for (int c = col_half; c < (rows + 7) / 8; c += 2) {
      uint32_t v[8];
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 8);
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (ok && out_col < p.N) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = c * 8 + i;
          if (m < rows) {
            if (kGrouped) {
              const int jrow = seg_lo + pass * pass_rows + m;          // sorted position of the row
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
    if (kGrouped && pass + 1 < n_pass) {                     // hand the accumulator back for the next pass
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) gb_mbar_arrive(acc_empty);
    }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
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

int umma_smem_bytes(int Mpad) {
  return 1024 + kSlabStages * (kASlabBytes + Mpad * 128) + kRawStages * kRawStageBytes + 4096 + 256;
}

// K slices: enough CTAs for the SMs when the layer has few 128-row tiles.
void umma_plan(int64_t N, int n_sb, int sms, int* slices, int* stages_per_slice) {
  const int tiles = (int)((N + kBM - 1) / kBM);
  const int n_raw = (n_sb + kRawSb - 1) / kRawSb;
  int want = sms / tiles;
  if (want < 1) want = 1;
  if (want > n_raw) want = n_raw;
  *stages_per_slice = (n_raw + want - 1) / want;
  *slices = (n_raw + *stages_per_slice - 1) / *stages_per_slice;
}

bool umma_applies(const gb_weight* w, int64_t M) {
  const gb_format& f = w->fmt;
  return M >= 2 && M <= kMaxRows && f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 &&
         f.scale_coding == GB_SCALE_V1 && f.type_size == kSbBytes && w->cb_row_offset == nullptr &&
         w->K >= 1024 && w->rows >= kBM && (w->row_stride % 16) == 0 && ((uintptr_t)w->qw & 15u) == 0 &&
         ((uintptr_t)w->codebook & 15u) == 0;
}

}  // namespace

int gb_prepare_umma() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)umma_decode_kernel<false>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, umma_smem_bytes(kMaxRows)));
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)umma_decode_kernel<true>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, umma_smem_bytes(kGroupRows)));
  return GB_OK;
}

int64_t gb_gemv_umma_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M < 2 || M > kMaxRows || K < 1024 || N < kBM) return 0;
  const int64_t xq = (M * K * 2 + 255) & ~255ll;
  int sms = gb_sm_count();
  if (sms <= 0) sms = 148;
  int slices, per;
  umma_plan(N, (int)(K / 256), sms, &slices, &per);
  return xq + (slices > 1 ? (int64_t)slices * M * N * 4 : 0);
}

int gb_gemv_umma(const void* x, int64_t M, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                 int64_t workspace_bytes, void* stream_) {
  if (!umma_applies(w, M) || ((uintptr_t)x & 15u) != 0 || act == GB_ACT_FP8_TOKEN) return GB_EUNSUPPORTED;
  const int sms = gb_sm_count();
  if (sms <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  const int64_t N = w->rows, K = w->K;
  UmmaParams p = {};
  p.N = N; p.K = K; p.M = (int)M; p.Mpad = (int)((M + 15) / 16 * 16);
  p.n_sb = (int)(K / 256);
  umma_plan(N, p.n_sb, sms, &p.slices, &p.stages_per_slice);
  const int64_t xq_bytes = act == GB_ACT_NONE ? 0 : ((M * K * 2 + 255) & ~255ll);
  const int64_t part_bytes = p.slices > 1 ? (int64_t)p.slices * M * N * 4 : 0;
  if (xq_bytes + part_bytes > 0 && (workspace == nullptr || workspace_bytes < xq_bytes + part_bytes))
    return gb_fail(GB_EWORKSPACE, "workspace of %lld bytes is too small (need %lld)", (long long)workspace_bytes,
                   (long long)(xq_bytes + part_bytes));
  const void* xin = x;
  if (act == GB_ACT_FP4_GROUP16) {
    int rc = gb_fp4_act_qdq(x, workspace, M, K, scale_rule, stream_);
    if (rc != GB_OK) return rc;
    xin = workspace;
  }
  CUtensorMap map_w, map_x;
  int rc = gb_tensor_map_bytes_2d(&map_w, w->qw, (uint64_t)p.n_sb * kSbBytes, (uint64_t)N, (uint64_t)w->row_stride,
                                  kSbBytes, kBM);
  if (rc != GB_OK) return rc;
  rc = gb_tensor_map_operand(&map_x, xin, M, K, 2, p.Mpad);
  if (rc != GB_OK) return rc;
  p.codebook = (const uint4*)w->codebook;
  p.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  p.y = (uint16_t*)y;
  p.partial = p.slices > 1 ? (float*)((uint8_t*)workspace + xq_bytes) : nullptr;
  // fp32 accumulate, bf16 x bf16, both K-major, N = activation rows (padded), M = 128 weight rows
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.Mpad >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.tmem_cols = 32;
  while ((int)p.tmem_cols < p.Mpad) p.tmem_cols <<= 1;
  p.status = gb_status_word();
  dim3 grid((unsigned)((N + kBM - 1) / kBM), (unsigned)p.slices);
  GB_CUDA_OK(gb_launch(umma_decode_kernel<false>, grid, dim3(kUmmaThreads), (size_t)umma_smem_bytes(p.Mpad),
                       (cudaStream_t)stream_, map_w, map_x, p));
  if (p.slices > 1) {
    const int64_t MN = M * N;
    GB_CUDA_OK(gb_launch(umma_finalize_kernel, dim3((unsigned)((MN + 255) / 256)), dim3(256), 0,
                         (cudaStream_t)stream_, (const float*)p.partial, p.slices, MN, p.global_scale,
                         (uint16_t*)y));
  }
  return GB_OK;
}

extern "C" {

int gb_moe_gemv_sorted(const void* x_sorted, const gb_weight* w, int64_t expert_stride, int64_t E,
                       const int32_t* seg_offsets, const int32_t* row_map, int64_t P, void* y,
                       const gb_peer_rows* y_rows, void* stream_) {
  GB_REQUIRE(x_sorted && w && seg_offsets && (y || y_rows), "null pointer argument");
  GB_REQUIRE(E >= 1 && P >= 0, "bad shape E=%lld P=%lld", (long long)E, (long long)P);
  int rc = gb_check_weight(w);
  if (rc != GB_OK) return rc;
  const gb_format& f = w->fmt;
  const int64_t N = w->rows, K = w->K;
  if (!(f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
        f.type_size == kSbBytes && w->cb_row_offset == nullptr && N % kBM == 0 && (w->row_stride % 16) == 0 &&
        expert_stride == N * w->row_stride && ((uintptr_t)w->qw & 15u) == 0 && ((uintptr_t)w->codebook & 15u) == 0 &&
        ((uintptr_t)x_sorted & 15u) == 0 && E * N < (1ll << 31)))
    return gb_fail(GB_EUNSUPPORTED, "the sorted-rows expert kernel takes contiguous stacks of the literal fp4 format with N %% 128 == 0");
  if (P == 0) return GB_OK;
  if (gb_sm_count() <= 0) return gb_fail(GB_ECUDA, "no usable CUDA device: %s", gb_last_error());
  UmmaParams p = {};
  p.N = N; p.K = K; p.M = kGroupRows; p.Mpad = kGroupRows;
  p.n_sb = (int)(K / 256);
  p.slices = 1;
  p.stages_per_slice = (p.n_sb + kRawSb - 1) / kRawSb;
  CUtensorMap map_w, map_x;
  rc = gb_tensor_map_bytes_2d(&map_w, w->qw, (uint64_t)p.n_sb * kSbBytes, (uint64_t)(E * N), (uint64_t)w->row_stride,
                              kSbBytes, kBM);
  if (rc != GB_OK) return rc;
  rc = gb_tensor_map_operand(&map_x, x_sorted, P, K, 2, kGroupRows);
  if (rc != GB_OK) return rc;
  p.codebook = (const uint4*)w->codebook;
  p.global_scale = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  p.y = (uint16_t*)y;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kGroupRows >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  p.tmem_cols = kGroupRows;
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
  dim3 grid((unsigned)(E * p.tiles_n), 1);
  GB_CUDA_OK(gb_launch(umma_decode_kernel<true>, grid, dim3(kUmmaThreads), (size_t)umma_smem_bytes(kGroupRows),
                       (cudaStream_t)stream_, map_w, map_x, p));
  return GB_OK;
}

}  // extern "C"
