// Routing and combine kernels of the routed-MoE path.
#include "gb_common.cuh"

namespace {

constexpr int kRouteThreads = 1024;

// One CTA: shared-memory histogram over experts, exclusive scan, then each warp
// fills whole experts in pair order with ballots, so the grouping is stable
// (token-ascending inside an expert) and identical from run to run.
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const int32_t* __restrict__ ids, int P, int E, int first_expert, int32_t* __restrict__ counts,
                 int32_t* __restrict__ offsets, int32_t* __restrict__ order,
                 const float* __restrict__ weights, float* __restrict__ pair_w) {
  extern __shared__ int32_t sh[];   // [E] counts, [E+1] offsets
  int32_t* cnt = sh;
  int32_t* off = sh + E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kRouteThreads / 32;
  gb_pdl_launch_dependents();
  for (int e = tid; e < E; e += kRouteThreads) cnt[e] = 0;
  gb_pdl_wait();
  __syncthreads();
  for (int i = tid; i < P; i += kRouteThreads) {
    const int id = ids[i] - first_expert;
    const bool live = id >= 0 && id < E;
    if (live) atomicAdd(&cnt[id], 1);
    // combine weight of the pair: the router weight rounded to bf16, zero for a dropped pair
    if (pair_w) pair_w[i] = live ? gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(weights[i])) : 0.0f;
  }
  __syncthreads();
  if (warp == 0) {
    // warp-wide exclusive scan over E in chunks of 32
    int running = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int v = e < E ? cnt[e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (e < E) off[e] = running + incl - v;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) off[E] = running;
  }
  __syncthreads();
  for (int e = tid; e < E; e += kRouteThreads) counts[e] = cnt[e];
  for (int e = tid; e <= E; e += kRouteThreads) offsets[e] = off[e];
  for (int i = off[E] + tid; i < P; i += kRouteThreads) order[i] = 0;   // dropped (padding) pairs
  for (int e = warp; e < E; e += nwarps) {
    if (cnt[e] == 0) continue;
    int pos = off[e];
    for (int base = 0; base < P; base += 32) {
      const int i = base + lane;
      const bool hit = i < P && ids[i] - first_expert == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) order[pos + __popc(mask & ((1u << lane) - 1u))] = i;
      pos += __popc(mask);
    }
  }
}

// out[t][h] = bf16( sum_slot w[t*topk+slot] * y[t*topk+slot][h] ), fp32 accumulate.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint16_t* __restrict__ y, const float* __restrict__ pair_w,
                   const int32_t* __restrict__ ids, int E, int topk, int64_t H, int round_w,
                   uint16_t* __restrict__ out) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  const int64_t t = blockIdx.y;
  const int64_t h2 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // pair of columns
  if (h2 * 2 >= H) return;
  float a0 = 0.f, a1 = 0.f;
  for (int s = 0; s < topk; ++s) {
    const int64_t p = t * topk + s;
    if (ids) {                      // a dropped pair has no output row: nothing was written there
      const int id = ids[p];
      if (id < 0 || id >= E) continue;
    }
    float w = pair_w[p];
    if (round_w) w = gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(w));
    const uint32_t v = *reinterpret_cast<const uint32_t*>(y + p * H + h2 * 2);
    a0 = fmaf(w, gb_bf16_bits_to_f32(v & 0xFFFFu), a0);
    a1 = fmaf(w, gb_bf16_bits_to_f32(v >> 16), a1);
  }
  *reinterpret_cast<uint32_t*>(out + t * H + h2 * 2) = gb_f32_to_bf16_bits(a0) | (gb_f32_to_bf16_bits(a1) << 16);
}

}  // namespace

extern "C" {

int gb_moe_route(const int32_t* topk_ids, int64_t T, int64_t topk, int64_t E, int64_t expert_base,
                 int32_t* counts, int32_t* offsets, int32_t* order, const float* topk_weights, float* pair_w, void* stream) {
  GB_REQUIRE(topk_ids && counts && offsets && order, "null pointer argument");
  GB_REQUIRE((topk_weights == nullptr) == (pair_w == nullptr), "topk_weights and pair_w go together");
  GB_REQUIRE(T >= 0 && topk >= 1 && E >= 1 && E <= 4096, "bad routing shape T=%lld topk=%lld E=%lld",
             (long long)T, (long long)topk, (long long)E);
  GB_REQUIRE(T * topk < (1ll << 30), "too many routed pairs");
  GB_CUDA_OK(gb_launch(moe_route_kernel, dim3(1), dim3(kRouteThreads), (size_t)(2 * E + 1) * sizeof(int32_t),
                       (cudaStream_t)stream, topk_ids, (int)(T * topk), (int)E, (int)expert_base, counts, offsets,
                       order, topk_weights, pair_w));
  return GB_OK;
}

int gb_moe_combine(const void* y, const float* pair_w, const int32_t* topk_ids, int64_t E, int64_t T,
                   int64_t topk, int64_t H, int round_weights, void* out, void* stream) {
  GB_REQUIRE(y && pair_w && out, "null pointer argument");
  GB_REQUIRE(T >= 0 && topk >= 1 && H > 0 && H % 2 == 0, "bad combine shape T=%lld topk=%lld H=%lld",
             (long long)T, (long long)topk, (long long)H);
  if (T == 0) return GB_OK;
  dim3 grid((unsigned)((H / 2 + 255) / 256), (unsigned)T);
  GB_CUDA_OK(gb_launch(moe_combine_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)y, pair_w,
                       topk_ids, (int)E, (int)topk, H, round_weights ? 1 : 0, (uint16_t*)out));
  return GB_OK;
}

}  // extern "C"
