// M = 1 linear for the literal format (fp4 grid, full mode, k = 8, E4M3-direct scales) by
// inner-product tables.
//
// With one 256-entry codebook and one activation row, a codeword's contribution to the dot
// product can only take 256 values per position: T[s][c][v] = <codebook[c], x[256 s + 8 v ..+8]>.
// A CTA owns four superblock columns of K and a band of rows.  It builds T for its columns
// once (tensor cores: codebook x activation segments, 128 KiB of fp32 in shared memory; the
// fp4 activation bucket is applied on the way in), then streams its rows' 192-byte slices
// through a TMA ring and spends, per 16 weights, two table lookups, one add and one scaled
// accumulate.  That is about 7 warp instructions and 4 shared-memory wavefronts per 48 packed
// bytes, against ~270 and ~80 for expanding every weight, which is what lets a 1.5-bit format
// approach the HBM stream.  Lanes 0..15 of a warp walk one row, lanes 16..31 the next; lane l
// owns group l (positions 2l, 2l+1) so its two lookups always fall in banks 2l and 2l+1, and
// the two half-warps take them in opposite order: no bank conflicts.
//
// K slices write their partial sums to their own slot; a second tiny kernel adds the slots,
// applies the global scale and rounds to bf16 once.
#include "gb_common.cuh"

#include <cuda.h>

namespace {

constexpr int kS = 4;                         // superblock columns per CTA
constexpr int kConsumers = 16;                // warps
constexpr int kDotThreads = (kConsumers + 1) * 32;
constexpr int kStageRows = 4 * kConsumers;    // 64 rows per stage, four per warp
constexpr int kRowBytes = kS * 48;            // 192 bytes of each row per stage
constexpr int kStageBytes = kStageRows * kRowBytes;
constexpr int kDotStages = 6;
constexpr int kTableFloats = kS * 256 * 32;
constexpr int kDotSmem = kTableFloats * 4 + kDotStages * kStageBytes + kS * 512 + 256 + 128;

struct DotParams {
  const uint16_t* x;        // [K] bf16
  const uint16_t* codebook; // [256 * 8] bf16
  int act, scale_rule;
  int64_t N;
  int n_sb, n_slices, n_groups, rows_per_group;
  float* ws;                // [n_slices][N] partial sums
  int* status;
};

GB_DEVINL float lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
GB_DEVINL uint32_t lds_b16(uint32_t a) {
  uint32_t v;
  asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
  return v;
}
// One superblock of one row for this lane's group: two table lookups, their sum, times the
// group's scale.  The scale byte is loaded sign-extended, so one shift and one mask put its
// exponent/mantissa into the fp32 fields (value * 2^-120, subnormal codes included) and its
// sign into bit 31; the table carries the compensating 2^100 so products stay normal.
GB_DEVINL float dot_superblock(uint32_t sbp, uint32_t tabA, uint32_t tabB, int l, uint32_t sel, float acc) {
  const uint32_t idx2 = __byte_perm(lds_b16(sbp + 2u * l), 0u, sel);       // (code A) | (code B) << 8
  const float tA = lds_f32(tabA + ((idx2 & 0xFFu) << 7));
  const float tB = lds_f32(tabB + ((idx2 >> 8) << 7));
  int32_t sc;
  asm volatile("ld.shared.s8 %0, [%1];" : "=r"(sc) : "r"(sbp + 32u + l));
  const float f = __uint_as_float(((uint32_t)sc << 20) & 0x87F00000u);
  return fmaf(tA + tB, f, acc);
}

__global__ void __launch_bounds__(kDotThreads, 1)
gemv_dot_kernel(const __grid_constant__ CUtensorMap map_w, const DotParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  float* table = reinterpret_cast<float*>(smem);
  uint8_t* ring = smem + kTableFloats * 4;
  uint16_t* xq = reinterpret_cast<uint16_t*>(ring + kDotStages * kStageBytes);      // kS * 256 bf16
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xq) + kS * 512);
  uint64_t* empty_bar = full_bar + kDotStages;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x % p.n_slices, group = blockIdx.x / p.n_slices;
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
            ::"r"(gb_smem_u32(ring + (size_t)s * kStageBytes)), "l"(reinterpret_cast<uint64_t>(&map_w)),
              "r"(sb0 * 48), "r"((int)(row_begin + (int64_t)st * kStageRows)), "r"(gb_smem_u32(&full_bar[s]))
            : "memory");
      }
    }
    return;
  }

  // ---- inner-product tables ----
  // One unit = one superblock column x eight codes x all 32 positions: two MMAs with the
  // activation segments as the 16 rows (A[m][k] = x[8 (16 h + m) + k], k < 8) and the eight
  // codewords as the columns (B[k][n] = codebook[c0 + n][k]).  Warp w owns code blocks 2w and
  // 2w + 1 for every column, so its two B fragments are loaded once, before the wait.
  const int g = lane >> 2, t = lane & 3;
  uint32_t bfrag[2];
  {
    const uint32_t* cb32 = reinterpret_cast<const uint32_t*>(p.codebook);
#pragma unroll
    for (int j = 0; j < 2; ++j) bfrag[j] = __ldg(cb32 + ((2 * warp + j) * 8 + g) * 4 + t);
  }

  // ---- this slice of the activation row, through its bucket, into shared memory ----
  gb_pdl_wait();                       // the activations (and the partial-sum slots) belong to earlier kernels
  if (tid < ns * 16) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (int64_t)sb0 * 256 + tid * 16);
    const uint4 r0 = src[0], r1 = src[1];
    uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    if (p.act == GB_ACT_FP4_GROUP16) gb_fp4_group16_qdq(w, p.scale_rule);
    uint4* dst = reinterpret_cast<uint4*>(xq + tid * 16);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

  {
    const uint32_t* xq32 = reinterpret_cast<const uint32_t*>(xq);
    for (int s = 0; s < ns; ++s) {
      uint32_t a[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a[h][0] = xq32[s * 128 + (16 * h + g) * 4 + t];
        a[h][1] = xq32[s * 128 + (16 * h + g + 8) * 4 + t];
        a[h][2] = 0u;
        a[h][3] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
        gb_mma_bf16_16816(d0, a[0], bfrag[j], 0u);      // positions g, g + 8
        gb_mma_bf16_16816(d1, a[1], bfrag[j], 0u);      // positions 16 + g, 24 + g
        // v[cc][pb]: code 2t + cc of the block, position 8 pb + g
        float v[2][4] = {{d0[0], d0[2], d1[0], d1[2]}, {d0[1], d0[3], d1[1], d1[3]}};
        // Store number q of a lane takes position block (t + q) & 3, so the four lanes that share
        // g write four different bank octets: every store instruction covers all 32 banks once.
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          if (t & 1) { const float x0 = v[cc][0]; v[cc][0] = v[cc][1]; v[cc][1] = v[cc][2]; v[cc][2] = v[cc][3]; v[cc][3] = x0; }
          if (t & 2) { const float x0 = v[cc][0], x1 = v[cc][1]; v[cc][0] = v[cc][2]; v[cc][1] = v[cc][3]; v[cc][2] = x0; v[cc][3] = x1; }
          float* row = table + ((s * 256 + (2 * warp + j) * 8 + 2 * t + cc) * 32 + g);
#pragma unroll
          for (int q = 0; q < 4; ++q) row[((t + q) & 3) * 8] = v[cc][q] * 0x1p100f;
        }
      }
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");

  // ---- stream the rows ----
  const int h = lane >> 4, l = lane & 15;
  // Half-warp 0 looks up position 2l then 2l+1, half-warp 1 the other way round (its two index
  // bytes are swapped once with a byte permute), so the 32 lanes of a lookup hit 32 banks.
  const uint32_t sel = h ? 0x4401u : 0x4410u;
  const uint32_t baseA = gb_smem_u32(table) + (uint32_t)(2 * l + h) * 4u;
  const uint32_t baseB = gb_smem_u32(table) + (uint32_t)(2 * l + 1 - h) * 4u;
  const uint32_t ring_s = gb_smem_u32(ring);
  float* my_ws = p.ws + (int64_t)slice * p.N;
  for (int st = 0; st < n_stages; ++st) {
    const int s = st % kDotStages;
    if (!gb_mbar_wait(&full_bar[s], (st / kDotStages) & 1)) atomicExch(p.status, 22);
#pragma unroll
    for (int step = 0; step < 2; ++step) {
      const int row_local = 4 * warp + 2 * step + h;
      const uint32_t rowp = ring_s + (uint32_t)s * kStageBytes + (uint32_t)row_local * kRowBytes;
      float acc = 0.f;
      if (ns == kS) {
#pragma unroll
        for (int sb = 0; sb < kS; ++sb) acc = dot_superblock(rowp + sb * 48, baseA + sb * 32768, baseB + sb * 32768, l, sel, acc);
      } else {
        for (int sb = 0; sb < ns; ++sb) acc = dot_superblock(rowp + sb * 48, baseA + sb * 32768, baseB + sb * 32768, l, sel, acc);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const int64_t row = row_begin + (int64_t)st * kStageRows + row_local;
      if (l == 0 && row < row_end) my_ws[row] = acc * 0x1p20f;       // table entries carry 2^100, scales 2^-120
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

}  // namespace

int gb_prepare_dot() {
  GB_CUDA_OK(cudaFuncSetAttribute((const void*)gemv_dot_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDotSmem));
  return GB_OK;
}

int64_t gb_gemv_dot_workspace_bytes(int64_t N, int64_t K) {
  const int64_t n_slices = (K / 256 + kS - 1) / kS;
  return n_slices * N * (int64_t)sizeof(float);
}

int gb_gemv_dot(const void* x, const gb_weight* w, int act, int scale_rule, void* y, void* workspace,
                int64_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const gb_format& f = w->fmt;
  const bool mine = f.grid == GB_GRID_FP4 && f.mode == GB_MODE_FULL && f.k_bits == 8 && f.scale_coding == GB_SCALE_V1 &&
                    w->cb_row_offset == nullptr && ((uintptr_t)w->qw & 15u) == 0 && w->row_stride % 16 == 0 &&
                    (act == GB_ACT_NONE || act == GB_ACT_FP4_GROUP16) && w->rows >= 512 && w->K >= 256 * kS &&
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
  GB_CUDA_OK(gb_launch(gemv_dot_kernel, dim3(p.n_slices * p.n_groups), dim3(kDotThreads), kDotSmem, stream, map, p));
  const float gs = w->global_scale == 0.0f ? 1.0f : w->global_scale;
  GB_CUDA_OK(gb_launch(dot_finalize_kernel, dim3((unsigned)((w->rows + 255) / 256)), dim3(256), 0, stream,
                       (const float*)p.ws, p.n_slices, (int64_t)w->rows, gs, (uint16_t*)y));
  return GB_OK;
}
