#include "host_util.h"
#include "nsa_b200_instrument.h"

#include <cudaTypedefs.h>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace nsa {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                 uint64_t stride1, uint64_t stride2, uint32_t b0, uint32_t b1, uint32_t b2) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return kUnsupported;
  if (!aligned16(base) || (stride1 * 2) % 16 || (stride2 * 2) % 16 || (b0 * 2) % 16) return kInvalid;
  cuuint64_t dims[3] = {n0, n1, n2};
  cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = (b0 * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kInvalid;
}

int make_tmap_4d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                 uint64_t n3, uint64_t stride1, uint64_t stride2, uint64_t stride3, uint32_t b0, uint32_t b2, uint32_t b3) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return kUnsupported;
  if (!aligned16(base) || (stride1 * 2) % 16 || (stride2 * 2) % 16 || (stride3 * 2) % 16 || (b0 * 2) % 16) return kInvalid;
  cuuint64_t dims[4] = {n0, n1, n2, n3};
  cuuint64_t strides[3] = {stride1 * 2, stride2 * 2, stride3 * 2};
  cuuint32_t box[4] = {b0, 1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapSwizzle sw = (b0 * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = g_encode(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kOk : kInvalid;
}

// One status word per device that loads the library (a module-scope device variable, zero at load).
__device__ int g_status_word;

static int* g_status[64] = {};
static std::mutex g_status_mu;

int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    g_status[dev] = static_cast<int*>(p);
  }
  return g_status[dev];
}

int read_status(cudaStream_t stream) {
  int* w = status_word();
  if (!w) return 0;
  int h = 0;
  if (cudaMemcpyAsync(&h, w, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return 0;
  cudaStreamSynchronize(stream);
  if (h) cudaMemsetAsync(w, 0, sizeof(int), stream);
  return h;
}

}  // namespace nsa

namespace nsa {
static std::atomic<long long> g_launches{0};
static bool g_prof_on = false;
struct Pending { std::string tag; cudaEvent_t a, b; };
static std::vector<Pending> g_pending;
static std::vector<cudaEvent_t> g_free_events;
static std::mutex g_prof_mu;

static cudaEvent_t get_event() {
  if (!g_free_events.empty()) { cudaEvent_t e = g_free_events.back(); g_free_events.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

void launch_begin(const char* tag, cudaStream_t stream) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  Pending pd{tag, get_event(), get_event()};
  cudaEventRecord(pd.a, stream);
  g_pending.push_back(pd);
}

void launch_end(cudaStream_t stream) {
  if (!g_prof_on) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!g_pending.empty()) cudaEventRecord(g_pending.back().b, stream);
}
}  // namespace nsa

extern "C" long long nsa_launch_count(void) { return nsa::g_launches.load(); }

extern "C" int nsa_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(nsa::g_prof_mu);
  nsa::g_prof_on = on != 0;
  return 0;
}

// Writes one line per kernel tag, "tag launches total_ms\n", for every launch recorded since the last call;
// synchronises the device.  Returns the number of bytes written (0 when nothing was recorded).
extern "C" int nsa_profile_collect(char* buf, int buflen) {
  using namespace nsa;
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lk(g_prof_mu);
  std::map<std::string, std::pair<long long, double>> acc;
  std::vector<std::string> order;
  for (auto& pd : g_pending) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pd.a, pd.b) == cudaSuccess) {
      if (!acc.count(pd.tag)) order.push_back(pd.tag);
      acc[pd.tag].first += 1;
      acc[pd.tag].second += ms;
    }
    g_free_events.push_back(pd.a);
    g_free_events.push_back(pd.b);
  }
  g_pending.clear();
  int n = 0;
  for (auto& t : order) {
    char line[160];
    const int len = snprintf(line, sizeof line, "%s %lld %.6f\n", t.c_str(), acc[t].first, acc[t].second);
    if (buf && n + len < buflen) { memcpy(buf + n, line, len); n += len; }
  }
  if (buf && n < buflen) buf[n] = 0;
  return n;
}

extern "C" int nsa_version(void) { return (0 << 16) | 1; }

extern "C" int nsa_last_device_status(void* stream) { return nsa::read_status(static_cast<cudaStream_t>(stream)); }
