// Process-wide pieces of the C ABI: error text, version, device properties.
#include "aps_common.cuh"

#include <initializer_list>

namespace aps {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

ProfileEvents* profile_events(int which) {
  static thread_local ProfileEvents ev[2] = {{nullptr, nullptr}, {nullptr, nullptr}};
  return &ev[which & 1];
}

}  // namespace aps

extern "C" int aps_set_profile_events(int which, void* start_event, void* stop_event) {
  if (which < 0 || which > 1) return aps::fail(APS_ERR_SHAPE, "set_profile_events: which must be 0 or 1");
  aps::ProfileEvents* ev = aps::profile_events(which);
  ev->start = static_cast<cudaEvent_t>(start_event);
  ev->stop = static_cast<cudaEvent_t>(stop_event);
  return APS_OK;
}

extern "C" const char* aps_last_error(void) { return aps::last_error_buffer(); }

extern "C" const char* aps_version(void) { return "aptserve_b200 0.1 (sm_100a)"; }
