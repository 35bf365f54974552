// Peer-memory exchange between the ranks of one NVSwitch node: buffers shared between the
// ranks' processes through CUDA IPC, an all-gather whose stores go straight into every
// peer's buffer over NVLink, and the cross-GPU barrier that opens and closes it.  The
// reference is single-GPU (gridbook/config.py:565-576); nothing here has a counterpart there.
//
// Flag block of a rank (GB_PEER_FLAG_BYTES, zero at allocation), as 32-bit words:
//   [0..7]   ready[r]: rank r has reached exchange number `epoch` (everything it enqueued
//            before that exchange, reads of the shared buffers included, has finished)
//   [8..15]  done[r]:  rank r's stores of exchange number `epoch` are visible
//   [16]     epoch of the last finished exchange (own use)
//   [17]     CTA arrival counter of the running exchange (own use)
//   [18]     number of the last finished flag-in-data exchange (own use)
//   [19]     CTA arrival counter of the running flag-in-data exchange (own use)
// Epochs only grow, and a waiter accepts any value at or past the one it waits for, so a
// fast peer that is already one exchange ahead never strands a slow one.  Every wait is
// bounded (two seconds unless gb_set_wait_limit_ms says otherwise); one that runs out raises the status word (value 3) and carries on.
#include "gb_common.cuh"

namespace {

constexpr int kMaxSeg = 4;

struct PeerSeg {
  const uint8_t* src;               // local source, first row
  uint8_t* dst[GB_PEER_MAX];        // destination of this rank's piece inside every rank's buffer
  int64_t rows, row_bytes, src_pitch, dst_pitch;
};

struct PeerParams {
  uint32_t* flags[GB_PEER_MAX];
  int rank, world, n_seg;
  PeerSeg seg[kMaxSeg];
  int* status;
  unsigned long long wait_ns;       // how long a wait may spin
};

GB_DEVINL void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
GB_DEVINL uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *slot has reached `epoch`; false once `limit_ns` have passed.
GB_DEVINL bool wait_epoch(const uint32_t* slot, uint32_t epoch, unsigned long long limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    if ((int32_t)(ld_acquire_sys(slot) - epoch) >= 0) return true;
    if ((spin & 63u) == 63u) {
      const uint64_t now = gb_globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}

// One launch per rank, the same sequence of launches on every rank.
//   1. tell every peer this rank has arrived; wait until every peer has (their buffers are free)
//   2. copy this rank's pieces into every rank's buffer (plain peer stores)
//   3. the last CTA to finish tells every peer the stores are visible and waits for theirs
// With n_seg == 0 only step 3 runs: "everything I stored before this launch is visible".
__global__ void __launch_bounds__(256) peer_exchange_kernel(const __grid_constant__ PeerParams p) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_last;
  uint32_t* mine = p.flags[p.rank];
  const int tid = threadIdx.x;
  gb_pdl_launch_dependents();
  gb_pdl_wait();                      // arriving here says: everything enqueued before has finished
  if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(mine + 16) + 1u;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (p.n_seg > 0) {                   // a plain barrier has no buffer to wait for
    if (tid < p.world) {
      if (blockIdx.x == 0) st_release_sys(p.flags[tid] + p.rank, epoch);
      if (!wait_epoch(mine + tid, epoch, p.wait_ns)) atomicExch(p.status, 3);
    }
    __syncthreads();
  }

  for (int s = 0; s < p.n_seg; ++s) {
    const PeerSeg& g = p.seg[s];
    const bool vec = ((g.row_bytes | g.src_pitch | g.dst_pitch | (int64_t)(uintptr_t)g.src) & 15) == 0;
    if (vec) {
      const int64_t per_row = g.row_bytes >> 4, per_peer = g.rows * per_row, total = per_peer * p.world;
      for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i / per_peer);
        const int64_t j = i - (int64_t)d * per_peer, r = j / per_row, c = j - r * per_row;
        const uint4 v = *reinterpret_cast<const uint4*>(g.src + r * g.src_pitch + c * 16);
        uint8_t* dst = g.dst[d] + r * g.dst_pitch + c * 16;
        if (((uintptr_t)dst & 15) == 0) {
          *reinterpret_cast<uint4*>(dst) = v;
        } else {                      // destination column offset not 16-byte aligned: 4-byte stores
          uint32_t* d4 = reinterpret_cast<uint32_t*>(dst);
          d4[0] = v.x; d4[1] = v.y; d4[2] = v.z; d4[3] = v.w;
        }
      }
    } else {                          // row_bytes and pitches are multiples of 4 (checked on the host)
      const int64_t per_row = g.row_bytes >> 2, per_peer = g.rows * per_row, total = per_peer * p.world;
      for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i / per_peer);
        const int64_t j = i - (int64_t)d * per_peer, r = j / per_row, c = j - r * per_row;
        *reinterpret_cast<uint32_t*>(g.dst[d] + r * g.dst_pitch + c * 4) =
            *reinterpret_cast<const uint32_t*>(g.src + r * g.src_pitch + c * 4);
      }
    }
  }

  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicAdd(mine + 17, 1u);
    s_last = (old == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (tid < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[tid] + 8 + p.rank, epoch);
    if (!wait_epoch(mine + 8 + tid, epoch, p.wait_ns)) atomicExch(p.status, 3);
  }
  __syncthreads();
  if (tid == 0) {
    mine[17] = 0u;
    mine[16] = epoch;
  }
}

// ---- flag-in-data all-gather ------------------------------------------------------------
// For small pieces the two flag round trips above cost more than the data.  Here every 4-byte
// word travels as an 8-byte store {word, exchange number} into a staging slot of the receiver,
// who spins on the number and unpacks into its own buffer: one one-way trip, no fence, no
// separate flag.  Slots alternate between two halves by the parity of the exchange number; a
// sender can only reach exchange e + 2 after it has received everybody's e + 1, which they sent
// after finishing e, so the half it overwrites has been read.
struct LLSeg {
  const uint8_t* src;
  uint8_t* dst_local[GB_PEER_MAX];   // where rank s's piece lands in this rank's buffer
  int64_t rows, row_words, src_pitch, dst_pitch, first_word;
};
struct LLParams {
  uint32_t* flags;                   // own flag block
  uint2* ll[GB_PEER_MAX];            // staging buffers, [parity][source rank][capacity]
  int64_t capacity, total_words;
  int rank, world, n_seg;
  LLSeg seg[kMaxSeg];
  int* status;
  unsigned long long wait_ns;
};

GB_DEVINL void st_ll(uint2* p, uint32_t word, uint32_t epoch) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(epoch) : "memory");
}
GB_DEVINL uint2 ld_ll(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) peer_ll_kernel(const __grid_constant__ LLParams p) {
  __shared__ uint32_t s_epoch;
  const int tid = threadIdx.x;
  gb_pdl_launch_dependents();
  gb_pdl_wait();
  if (tid == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(p.flags + 18) + 1u;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int64_t half = (int64_t)(epoch & 1u) * p.world * p.capacity;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // send: my words to every peer's staging slot, my own piece straight to its place
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < p.total_words; i += stride) {
    int s = 0;
    while (s + 1 < p.n_seg && i >= p.seg[s + 1].first_word) ++s;
    const LLSeg& g = p.seg[s];
    const int64_t j = i - g.first_word, r = j / g.row_words, c = j - r * g.row_words;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(g.src + r * g.src_pitch + c * 4);
    *reinterpret_cast<uint32_t*>(g.dst_local[p.rank] + r * g.dst_pitch + c * 4) = word;
    for (int d = 0; d < p.world; ++d)
      if (d != p.rank) st_ll(p.ll[d] + half + (int64_t)p.rank * p.capacity + i, word, epoch);
  }
  // receive: everybody else's words out of my staging slots
  bool late = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < p.total_words; i += stride) {
    int s = 0;
    while (s + 1 < p.n_seg && i >= p.seg[s + 1].first_word) ++s;
    const LLSeg& g = p.seg[s];
    const int64_t j = i - g.first_word, r = j / g.row_words, c = j - r * g.row_words;
    // all sources' slots are read at once; only those not there yet are polled
    const uint2* slot0 = p.ll[p.rank] + half + i;
    uint2 v[GB_PEER_MAX];
#pragma unroll
    for (int src = 0; src < GB_PEER_MAX; ++src)
      if (src < p.world && src != p.rank) v[src] = ld_ll(slot0 + (int64_t)src * p.capacity);
#pragma unroll
    for (int src = 0; src < GB_PEER_MAX; ++src) {
      if (src >= p.world || src == p.rank) continue;
      uint64_t t0 = 0;
      for (uint32_t spin = 0; v[src].y != epoch && !late; ++spin) {
        v[src] = ld_ll(slot0 + (int64_t)src * p.capacity);
        if ((spin & 63u) == 63u) {
          const uint64_t now = gb_globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > p.wait_ns) late = true;
        }
      }
      *reinterpret_cast<uint32_t*>(g.dst_local[src] + r * g.dst_pitch + c * 4) = v[src].x;
    }
  }
  if (late) atomicExch(p.status, 3);
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicAdd(p.flags + 19, 1u);
    if (old == gridDim.x - 1) {       // every CTA has read the exchange number by now
      p.flags[19] = 0u;
      p.flags[18] = epoch;
    }
  }
}

int check_group(const gb_peer_group* g) {
  GB_REQUIRE(g != nullptr, "null peer group");
  GB_REQUIRE(g->world >= 1 && g->world <= GB_PEER_MAX && g->rank >= 0 && g->rank < g->world,
             "bad peer group rank %d of %d", g->rank, g->world);
  for (int r = 0; r < g->world; ++r) GB_REQUIRE(g->flags[r] != nullptr, "peer group: flag block of rank %d is null", r);
  return GB_OK;
}

}  // namespace

extern "C" {

int gb_peer_alloc(int64_t bytes, void** ptr) {
  GB_REQUIRE(ptr != nullptr && bytes > 0, "bad peer allocation of %lld bytes", (long long)bytes);
  void* p = nullptr;
  GB_CUDA_OK(cudaMalloc(&p, (size_t)bytes));
  cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    return gb_fail(GB_ECUDA, "clearing a peer buffer: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return GB_OK;
}

int gb_peer_free(void* ptr) {
  if (ptr) GB_CUDA_OK(cudaFree(ptr));
  return GB_OK;
}

int gb_peer_export(void* ptr, void* handle64) {
  GB_REQUIRE(ptr && handle64, "null pointer argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == GB_PEER_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  GB_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, sizeof(h));
  return GB_OK;
}

int gb_peer_open(const void* handle64, void** ptr) {
  GB_REQUIRE(ptr && handle64, "null pointer argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  GB_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return GB_OK;
}

int gb_peer_close(void* ptr) {
  if (ptr) GB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return GB_OK;
}

int gb_peer_allgather(const gb_peer_group* g, const gb_peer_piece* pieces, int n_pieces, void* stream) {
  int rc = check_group(g);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(n_pieces >= 0 && n_pieces <= kMaxSeg, "at most %d pieces per exchange, got %d", kMaxSeg, n_pieces);
  GB_REQUIRE(n_pieces == 0 || pieces != nullptr, "null piece list");
  PeerParams p = {};
  p.rank = g->rank;
  p.world = g->world;
  p.n_seg = n_pieces;
  p.status = gb_status_word();
  p.wait_ns = gb_wait_limit_ns();
  for (int r = 0; r < g->world; ++r) p.flags[r] = (uint32_t*)g->flags[r];
  int64_t bytes = 0;
  for (int s = 0; s < n_pieces; ++s) {
    const gb_peer_piece& q = pieces[s];
    GB_REQUIRE(q.src && q.rows >= 0 && q.row_bytes >= 0, "piece %d: bad source", s);
    GB_REQUIRE(((q.row_bytes | q.src_pitch | q.dst_pitch | (int64_t)(uintptr_t)q.src) & 3) == 0,
               "piece %d: rows, pitches and pointers must be multiples of four bytes", s);
    p.seg[s].src = (const uint8_t*)q.src;
    p.seg[s].rows = q.rows;
    p.seg[s].row_bytes = q.row_bytes;
    p.seg[s].src_pitch = q.src_pitch;
    p.seg[s].dst_pitch = q.dst_pitch;
    for (int r = 0; r < g->world; ++r) {
      GB_REQUIRE(q.dst[r] != nullptr && ((uintptr_t)q.dst[r] & 3) == 0, "piece %d: bad destination on rank %d", s, r);
      p.seg[s].dst[r] = (uint8_t*)q.dst[r];
    }
    bytes += q.rows * q.row_bytes * g->world;
  }
  int grid = (int)((bytes / 16 + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 32) grid = 32;          // all CTAs resident at once; 32 saturate the links at these sizes
  GB_CUDA_OK(gb_launch(peer_exchange_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p));
  return GB_OK;
}

int gb_peer_allgather_ll(const gb_peer_group* g, void* const* ll, int64_t ll_bytes, const gb_peer_ll_piece* pieces,
                         int n_pieces, void* stream) {
  int rc = check_group(g);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(ll != nullptr && pieces != nullptr && n_pieces >= 1 && n_pieces <= kMaxSeg,
             "flag-in-data all-gather takes 1..%d pieces, got %d", kMaxSeg, n_pieces);
  LLParams p = {};
  p.rank = g->rank;
  p.world = g->world;
  p.n_seg = n_pieces;
  p.flags = (uint32_t*)g->flags[g->rank];
  p.status = gb_status_word();
  p.wait_ns = gb_wait_limit_ns();
  p.capacity = ll_bytes / (2 * (int64_t)g->world * 8);
  for (int r = 0; r < g->world; ++r) {
    GB_REQUIRE(ll[r] != nullptr && ((uintptr_t)ll[r] & 7) == 0, "staging buffer of rank %d is null or misaligned", r);
    p.ll[r] = (uint2*)ll[r];
  }
  int64_t words = 0;
  for (int s = 0; s < n_pieces; ++s) {
    const gb_peer_ll_piece& q = pieces[s];
    GB_REQUIRE(q.src && q.rows >= 0 && q.row_bytes >= 0, "piece %d: bad source", s);
    GB_REQUIRE(((q.row_bytes | q.src_pitch | q.dst_pitch | (int64_t)(uintptr_t)q.src) & 3) == 0,
               "piece %d: rows, pitches and pointers must be multiples of four bytes", s);
    p.seg[s].src = (const uint8_t*)q.src;
    p.seg[s].rows = q.rows;
    p.seg[s].row_words = q.row_bytes / 4;
    p.seg[s].src_pitch = q.src_pitch;
    p.seg[s].dst_pitch = q.dst_pitch;
    p.seg[s].first_word = words;
    for (int r = 0; r < g->world; ++r) {
      GB_REQUIRE(q.dst_local[r] != nullptr && ((uintptr_t)q.dst_local[r] & 3) == 0,
                 "piece %d: bad local destination for rank %d", s, r);
      p.seg[s].dst_local[r] = (uint8_t*)q.dst_local[r];
    }
    words += q.rows * (q.row_bytes / 4);
  }
  GB_REQUIRE(words <= p.capacity, "%lld words per rank exceed the staging capacity of %lld; use gb_peer_allgather",
             (long long)words, (long long)p.capacity);
  p.total_words = words;
  int grid = (int)((words + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > 64) grid = 64;
  GB_CUDA_OK(gb_launch(peer_ll_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p));
  return GB_OK;
}

int gb_peer_barrier(const gb_peer_group* g, void* stream) { return gb_peer_allgather(g, nullptr, 0, stream); }

}  // extern "C"
