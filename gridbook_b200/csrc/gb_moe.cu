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
                 const float* __restrict__ weights, float* __restrict__ pair_w, int tiled) {
  extern __shared__ int32_t sh[];   // [E] counts, [E+1] offsets; tiled: + [E][32] + [E]
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
  if (!tiled) {
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
    return;
  }
  // Many pairs: walk them in tiles of one pair per thread, in pair order.  Inside a tile a pair's
  // place among its expert's pairs = (pairs of that expert in earlier warps) + (its rank among
  // the warp's lanes with the same expert); wcnt[e][w] holds warp w's count, then its start.
  int32_t* wcnt = off + E + 1;            // [E][32]
  int32_t* cursor = wcnt + E * nwarps;    // [E] next free place of every expert
  for (int e = tid; e < E; e += kRouteThreads) cursor[e] = off[e];
  int next_raw = tid < P ? ids[tid] : -1;               // the next tile's id is loaded a tile ahead
  for (int base = 0; base < P; base += kRouteThreads) {
    for (int k = tid; k < E * nwarps; k += kRouteThreads) wcnt[k] = 0;
    const int i = base + tid;
    const int raw = next_raw;
    next_raw = i + kRouteThreads < P ? ids[i + kRouteThreads] : -1;
    __syncthreads();
    int id = -1;
    if (i < P) {
      const int v = raw - first_expert;
      if (v >= 0 && v < E) id = v;
    }
    const unsigned same = __match_any_sync(0xffffffffu, id);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (id >= 0 && rank == 0) wcnt[id * nwarps + warp] = __popc(same);
    __syncthreads();
    for (int e = warp; e < E; e += nwarps) {          // lane w scans warp w's count of expert e
      const int v = wcnt[e * nwarps + lane];
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      const int start = cursor[e];
      wcnt[e * nwarps + lane] = start + incl - v;
      __syncwarp();
      if (lane == 31) cursor[e] = start + incl;
    }
    __syncthreads();
    if (id >= 0) order[wcnt[id * nwarps + warp] + rank] = i;
    __syncthreads();
  }
}

// ---- routing over many pairs: three launches that use the whole GPU ---------------------
// Tiles of 1024 pairs.  (1) every tile counts its pairs per expert; (2) one CTA turns the counts
// into per-expert totals, segment offsets and, per tile, the number of an expert's pairs in
// earlier tiles; (3) every tile places its pairs: segment start + pairs in earlier tiles + pairs
// of that expert in earlier warps of the tile + rank among the warp's lanes with the same
// expert.  The same stable expert-major order as the one-CTA kernel.
__global__ void __launch_bounds__(kRouteThreads)
route_hist_kernel(const int32_t* __restrict__ ids, int P, int E, int first_expert, int32_t* __restrict__ hist,
                  const float* __restrict__ weights, float* __restrict__ pair_w) {
  extern __shared__ int32_t sh[];   // [E]
  gb_pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += kRouteThreads) sh[e] = 0;
  gb_pdl_wait();                    // nothing is written before the launch ahead has finished
  __syncthreads();
  const int i = blockIdx.x * kRouteThreads + threadIdx.x;
  if (i < P) {
    const int id = ids[i] - first_expert;
    const bool live = id >= 0 && id < E;
    if (live) atomicAdd(&sh[id], 1);
    if (pair_w) pair_w[i] = live ? gb_bf16_bits_to_f32(gb_f32_to_bf16_bits(weights[i])) : 0.0f;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kRouteThreads) hist[(int64_t)blockIdx.x * E + e] = sh[e];
}

__global__ void __launch_bounds__(kRouteThreads)
route_scan_kernel(int32_t* __restrict__ hist, int tiles, int P, int E, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ order) {
  extern __shared__ int32_t sh[];   // [E] counts, [E+1] offsets
  int32_t* cnt = sh;
  int32_t* off = sh + E;
  const int tid = threadIdx.x, lane = tid & 31;
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  for (int e = tid >> 5; e < E; e += kRouteThreads / 32) {   // a warp per expert, lanes over tiles
    int run = 0;
    for (int t0 = 0; t0 < tiles; t0 += 32) {     // exclusive prefix over the tiles, in place
      const int t = t0 + lane;
      const int v = t < tiles ? hist[(int64_t)t * E + e] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (t < tiles) hist[(int64_t)t * E + e] = run + incl - v;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) cnt[e] = run;
  }
  __syncthreads();
  if (tid < 32) {
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
}

__global__ void __launch_bounds__(kRouteThreads)
route_scatter_kernel(const int32_t* __restrict__ ids, int P, int E, int first_expert,
                     const int32_t* __restrict__ hist, const int32_t* __restrict__ offsets,
                     int32_t* __restrict__ order) {
  extern __shared__ int32_t wcnt[];   // [E][32]: warp w's count of expert e, then its start
  constexpr int nwarps = kRouteThreads / 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  gb_pdl_launch_dependents();
  for (int k = tid; k < E * nwarps; k += kRouteThreads) wcnt[k] = 0;
  gb_pdl_wait();
  const int i = blockIdx.x * kRouteThreads + tid;
  int id = -1;
  if (i < P) {
    const int v = ids[i] - first_expert;
    if (v >= 0 && v < E) id = v;
  }
  __syncthreads();
  const unsigned same = __match_any_sync(0xffffffffu, id);
  const int rank = __popc(same & ((1u << lane) - 1u));
  if (id >= 0 && rank == 0) wcnt[id * nwarps + warp] = __popc(same);
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    const int v = wcnt[e * nwarps + lane];
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += n;
    }
    wcnt[e * nwarps + lane] = offsets[e] + hist[(int64_t)blockIdx.x * E + e] + incl - v;
  }
  __syncthreads();
  if (id >= 0) order[wcnt[id * nwarps + warp] + rank] = i;
}

// Optional cross-GPU part of the combine (expert parallelism): before any row of y is read,
// tell every peer "my stores into your buffers are visible" and wait for the same from them
// (the second half of the exchange protocol in gb_peer.cu: flag words 8..15, exchange number in
// word 16, CTA counter in word 17).
struct CombinePeers {
  uint32_t* flags[GB_PEER_MAX];
  int rank, world;       // world == 0: no exchange
  int* status;
};

// out[t][h] = bf16( sum_slot w[t*topk+slot] * y[t*topk+slot][h] ), fp32 accumulate.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint16_t* __restrict__ y, const float* __restrict__ pair_w,
                   const int32_t* __restrict__ ids, int E, int topk, int64_t H, int round_w,
                   uint16_t* __restrict__ out, const __grid_constant__ CombinePeers peers) {
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  if (peers.world > 0) {
    __shared__ uint32_t s_epoch;
    uint32_t* mine = peers.flags[peers.rank];
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(mine + 16) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    if ((int)threadIdx.x < peers.world) {
      const int d = threadIdx.x;
      if (blockIdx.x == 0 && blockIdx.y == 0) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[d] + 8 + peers.rank), "r"(epoch) : "memory");
      }
      uint64_t t0 = 0;
      for (uint32_t spin = 0;; ++spin) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + 8 + d) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        if ((spin & 63u) == 63u) {
          const uint64_t now = gb_globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > 2000000000ull) { atomicExch(peers.status, 3); break; }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned total = gridDim.x * gridDim.y;
      const unsigned old = atomicAdd(mine + 17, 1u);
      if (old == total - 1) {          // every CTA has read the exchange number by now
        mine[17] = 0u;
        mine[16] = epoch;
      }
    }
  }
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

int64_t gb_moe_route_workspace_bytes(int64_t T, int64_t topk, int64_t E) {
  const int64_t P = T * topk;
  if (P < 4096 || E > 256 || E < 1) return 0;                 // the one-CTA kernel needs none
  return ((P + kRouteThreads - 1) / kRouteThreads) * E * (int64_t)sizeof(int32_t);
}

int gb_moe_route_ws(const int32_t* topk_ids, int64_t T, int64_t topk, int64_t E, int64_t expert_base,
                    int32_t* counts, int32_t* offsets, int32_t* order, const float* topk_weights, float* pair_w,
                    void* workspace, int64_t ws_bytes, void* stream) {
  GB_REQUIRE(topk_ids && counts && offsets && order, "null pointer argument");
  GB_REQUIRE((topk_weights == nullptr) == (pair_w == nullptr), "topk_weights and pair_w go together");
  GB_REQUIRE(T >= 0 && topk >= 1 && E >= 1 && E <= 4096, "bad routing shape T=%lld topk=%lld E=%lld",
             (long long)T, (long long)topk, (long long)E);
  GB_REQUIRE(T * topk < (1ll << 30), "too many routed pairs");
  const int64_t need = gb_moe_route_workspace_bytes(T, topk, E);
  cudaStream_t st = (cudaStream_t)stream;
  if (need > 0 && workspace != nullptr) {
    if (ws_bytes < need) return gb_fail(GB_EWORKSPACE, "routing workspace: %lld bytes given, %lld needed",
                                        (long long)ws_bytes, (long long)need);
    GB_REQUIRE(((uintptr_t)workspace & 3u) == 0, "routing workspace must be 4-byte aligned");
    const int P = (int)(T * topk), tiles = (P + kRouteThreads - 1) / kRouteThreads;
    int32_t* hist = (int32_t*)workspace;
    GB_CUDA_OK(gb_launch(route_hist_kernel, dim3(tiles), dim3(kRouteThreads), (size_t)E * sizeof(int32_t), st,
                         topk_ids, P, (int)E, (int)expert_base, hist, topk_weights, pair_w));
    GB_CUDA_OK(gb_launch(route_scan_kernel, dim3(1), dim3(kRouteThreads), (size_t)(2 * E + 1) * sizeof(int32_t), st,
                         hist, tiles, P, (int)E, counts, offsets, order));
    GB_CUDA_OK(gb_launch(route_scatter_kernel, dim3(tiles), dim3(kRouteThreads),
                         (size_t)E * (kRouteThreads / 32) * sizeof(int32_t), st, topk_ids, P, (int)E,
                         (int)expert_base, (const int32_t*)hist, (const int32_t*)offsets, order));
    return GB_OK;
  }
  // a warp per expert scanning all pairs costs E*P; from a few thousand pairs on, tiles of
  // 1024 pairs in pair order are cheaper (the per-warp counts need E*33 words of shared memory)
  const int tiled = T * topk >= 4096 && E <= 256;
  const size_t smem = (size_t)(2 * E + 1 + (tiled ? E * (kRouteThreads / 32 + 1) : 0)) * sizeof(int32_t);
  GB_CUDA_OK(gb_launch(moe_route_kernel, dim3(1), dim3(kRouteThreads), smem, st, topk_ids,
                       (int)(T * topk), (int)E, (int)expert_base, counts, offsets, order, topk_weights, pair_w,
                       tiled));
  return GB_OK;
}

int gb_moe_route(const int32_t* topk_ids, int64_t T, int64_t topk, int64_t E, int64_t expert_base,
                 int32_t* counts, int32_t* offsets, int32_t* order, const float* topk_weights, float* pair_w, void* stream) {
  return gb_moe_route_ws(topk_ids, T, topk, E, expert_base, counts, offsets, order, topk_weights, pair_w, nullptr, 0,
                         stream);
}

static int combine_launch(const void* y, const float* pair_w, const int32_t* topk_ids, int64_t E, int64_t T,
                          int64_t topk, int64_t H, int round_weights, void* out, const gb_peer_group* g, void* stream) {
  GB_REQUIRE(y && pair_w && out, "null pointer argument");
  GB_REQUIRE(T >= 0 && topk >= 1 && H > 0 && H % 2 == 0, "bad combine shape T=%lld topk=%lld H=%lld",
             (long long)T, (long long)topk, (long long)H);
  CombinePeers peers = {};
  if (g) {
    GB_REQUIRE(g->world >= 1 && g->world <= GB_PEER_MAX && g->rank >= 0 && g->rank < g->world, "bad peer group");
    GB_REQUIRE(T > 0, "the combine that closes an exchange needs at least one token");
    for (int r = 0; r < g->world; ++r) {
      GB_REQUIRE(g->flags[r] != nullptr, "peer group: flag block of rank %d is null", r);
      peers.flags[r] = (uint32_t*)g->flags[r];
    }
    peers.rank = g->rank;
    peers.world = g->world;
    peers.status = gb_status_word();
  }
  if (T == 0) return GB_OK;
  dim3 grid((unsigned)((H / 2 + 255) / 256), (unsigned)T);
  GB_CUDA_OK(gb_launch(moe_combine_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)y, pair_w,
                       topk_ids, (int)E, (int)topk, H, round_weights ? 1 : 0, (uint16_t*)out, peers));
  return GB_OK;
}

int gb_moe_combine(const void* y, const float* pair_w, const int32_t* topk_ids, int64_t E, int64_t T,
                   int64_t topk, int64_t H, int round_weights, void* out, void* stream) {
  return combine_launch(y, pair_w, topk_ids, E, T, topk, H, round_weights, out, nullptr, stream);
}

int gb_moe_combine_peer(const void* y, const float* pair_w, const int32_t* topk_ids, int64_t E, int64_t T,
                        int64_t topk, int64_t H, int round_weights, void* out, const gb_peer_group* g, void* stream) {
  GB_REQUIRE(g != nullptr, "null peer group");
  return combine_launch(y, pair_w, topk_ids, E, T, topk, H, round_weights, out, g, stream);
}

}  // extern "C"
