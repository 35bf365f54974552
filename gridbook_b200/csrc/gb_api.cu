// Host-side plumbing shared by every entry point: error text, per-device
// set-up, argument validation.
#include "gb_common.cuh"

#include <atomic>

#include <mutex>
#include <string.h>

namespace {
thread_local char g_error[512] = "";
std::mutex g_mutex;
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
int* g_status[kMaxDevices] = {nullptr};
}  // namespace

__device__ int g_gb_status_word = 0;

void gb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int gb_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

static int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

static int prepare_locked(int dev) {
  if (g_sm_count[dev] > 0) return GB_OK;
  int sms = 0;
  GB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int major = 0;
  GB_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    return gb_fail(GB_EUNSUPPORTED, "device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
  void* p = nullptr;
  GB_CUDA_OK(cudaGetSymbolAddress(&p, g_gb_status_word));
  g_status[dev] = (int*)p;
  g_sm_count[dev] = sms;
  return GB_OK;
}

static std::atomic<long long> g_launches{0};
void gb_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" int64_t gb_launch_count() { return (int64_t)g_launches.load(std::memory_order_relaxed); }

static std::atomic<unsigned long long> g_wait_ns{2000000000ull};
unsigned long long gb_wait_limit_ns() { return g_wait_ns.load(std::memory_order_relaxed); }

bool gb_pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("GRIDBOOK_B200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

int gb_sm_count() {
  const int dev = current_device_slot();
  if (dev < 0) return 0;
  if (g_sm_count[dev] == 0) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (prepare_locked(dev) != GB_OK) return 0;
  }
  return g_sm_count[dev];
}

int* gb_status_word() {
  const int dev = current_device_slot();
  if (dev < 0 || gb_sm_count() == 0) return nullptr;
  return g_status[dev];
}

int gb_check_format(const gb_format& f, int64_t K) {
  GB_REQUIRE(K > 0 && K % 256 == 0, "K=%lld must be a positive multiple of 256", (long long)K);
  GB_REQUIRE(f.grid == GB_GRID_FP4 || f.grid == GB_GRID_FP8, "unknown grid %d", f.grid);
  GB_REQUIRE(f.mode >= GB_MODE_PRODUCT && f.mode <= GB_MODE_FULL, "unknown mode %d", f.mode);
  if (f.mode == GB_MODE_PRODUCT) {
    GB_REQUIRE(f.n_sub == 2 || f.n_sub == 4, "product mode wants n_sub 2 or 4, got %d", f.n_sub);
    GB_REQUIRE(f.k_bits >= f.n_sub && f.k_bits <= 48, "k_bits %d out of range", f.k_bits);
    GB_REQUIRE((f.k_bits + f.n_sub - 1) / f.n_sub <= 14, "sub-table of 2^%d rows is too large",
               (f.k_bits + f.n_sub - 1) / f.n_sub);
  } else if (f.mode == GB_MODE_SIGNED) {
    GB_REQUIRE(f.k_bits >= 9 && f.k_bits <= 22, "signed mode wants 9 <= k_bits <= 22, got %d", f.k_bits);
  } else {
    GB_REQUIRE(f.k_bits >= 1 && f.k_bits <= 14, "full mode wants 1 <= k_bits <= 14, got %d", f.k_bits);
  }
  int scale_bytes = 0;
  if (f.grid == GB_GRID_FP4) {
    GB_REQUIRE(f.scale_coding == GB_SCALE_V1 || f.scale_coding == GB_SCALE_V2,
               "fp4 grid wants scale coding v1 or v2, got %d", f.scale_coding);
    scale_bytes = f.scale_coding == GB_SCALE_V1 ? 16 : 9;
  } else {
    GB_REQUIRE(f.scale_coding == GB_SCALE_NONE, "fp8 grid carries no scale plane");
  }
  // The superblock stride may exceed the packed bytes by up to 15 (padding after the scale plane,
  // ignored by every kernel): a host that wants 16-byte superblocks pads once at load.
  GB_REQUIRE(f.type_size >= 4 * f.k_bits + scale_bytes && f.type_size <= 4 * f.k_bits + scale_bytes + 15,
             "type_size %d does not match 4*%d+%d (plus at most 15 padding bytes) for this grid/scale coding",
             f.type_size, f.k_bits, scale_bytes);
  return GB_OK;
}

int gb_check_weight(const gb_weight* w) {
  GB_REQUIRE(w != nullptr, "null weight descriptor");
  int rc = gb_check_format(w->fmt, w->K);
  if (rc != GB_OK) return rc;
  GB_REQUIRE(w->qw != nullptr && w->codebook != nullptr, "null packed weights or codebook");
  GB_REQUIRE(w->rows > 0, "rows=%lld", (long long)w->rows);
  GB_REQUIRE(w->row_stride >= (w->K / 256) * w->fmt.type_size,
             "row stride %lld is shorter than the packed row (%lld bytes)",
             (long long)w->row_stride, (long long)((w->K / 256) * w->fmt.type_size));
  if (w->fmt.grid == GB_GRID_FP8)
    GB_REQUIRE(w->weight_scale != nullptr, "fp8 grid needs the per-row weight_scale");
  if (w->fmt.scale_coding == GB_SCALE_V2)
    GB_REQUIRE(w->compose != nullptr, "two-tier scale coding needs the compose table");
  return GB_OK;
}

extern "C" {

int gb_abi_version(void) { return GB_ABI_VERSION; }

const char* gb_last_error(void) { return g_error; }

int gb_prepare(int device) {
  GB_REQUIRE(device >= 0 && device < kMaxDevices, "device %d out of range", device);
  int prev = 0;
  GB_CUDA_OK(cudaGetDevice(&prev));
  GB_CUDA_OK(cudaSetDevice(device));
  int rc;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    rc = prepare_locked(device);
  }
  if (rc == GB_OK) rc = gb_prepare_kernels();
  if (rc == GB_OK) rc = gb_prepare_gemm();
  if (rc == GB_OK) rc = gb_prepare_dot();
  if (rc == GB_OK) rc = gb_prepare_umma();
  if (rc == GB_OK) rc = gb_prepare_tab();
  if (rc == GB_OK) rc = gb_prepare_gemm_fp4();
  cudaSetDevice(prev);
  return rc;
}

int gb_device_status(int device, int* status_out) {
  GB_REQUIRE(status_out != nullptr, "null status_out");
  GB_REQUIRE(device >= 0 && device < kMaxDevices && g_status[device] != nullptr,
             "device %d was not prepared", device);
  GB_CUDA_OK(cudaMemcpy(status_out, g_status[device], sizeof(int), cudaMemcpyDeviceToHost));
  return GB_OK;
}

int gb_device_status_reset(int device) {
  GB_REQUIRE(device >= 0 && device < kMaxDevices && g_status[device] != nullptr, "device %d was not prepared", device);
  const int zero = 0;
  GB_CUDA_OK(cudaMemcpy(g_status[device], &zero, sizeof(int), cudaMemcpyHostToDevice));
  return GB_OK;
}

int gb_set_wait_limit_ms(int ms) {
  GB_REQUIRE(ms >= 0 && ms <= 60000, "wait limit of %d ms is out of range (0 restores the default)", ms);
  g_wait_ns.store(ms == 0 ? 2000000000ull : (unsigned long long)ms * 1000000ull, std::memory_order_relaxed);
  return GB_OK;
}

}  // extern "C"
