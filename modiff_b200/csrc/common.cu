// Error reporting, device info and buffer-size helpers of the C ABI.
#include "common.cuh"

#include <string.h>

namespace modiff {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int validate_geom(const modiff_conv_geom* g) {
  MODIFF_CHECK_ARG(g != nullptr, "geometry pointer is NULL");
  MODIFF_CHECK_ARG(g->batch > 0 && g->cin > 0 && g->cout > 0, "batch/cin/cout must be positive");
  MODIFF_CHECK_ARG(g->h > 0 && g->w > 0 && g->kh > 0 && g->kw > 0, "spatial sizes must be positive");
  MODIFF_CHECK_ARG(g->stride == 1 || g->stride == 2, "stride %d unsupported (1 or 2)", g->stride);
  MODIFF_CHECK_ARG(g->pad_t >= 0 && g->pad_l >= 0 && g->pad_b >= 0 && g->pad_r >= 0,
                   "negative padding");
  MODIFF_CHECK_ARG(g->h + g->pad_t + g->pad_b >= g->kh && g->w + g->pad_l + g->pad_r >= g->kw,
                   "kernel larger than padded input");
  MODIFF_CHECK_ARG(g->split >= 0 && g->split < g->cin, "split %d outside [0, cin)", g->split);
  MODIFF_CHECK_ARG(g->split % 4 == 0, "split %d must be a multiple of 4", g->split);
  return MODIFF_OK;
}

}  // namespace modiff

using namespace modiff;

extern "C" {

int modiff_version(void) { return 100; }

const char* modiff_last_error(void) { return error_buffer(); }

int modiff_device_info(int* sm_count, int* cc_major, int* cc_minor) {
  int dev = 0;
  MODIFF_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp p;
  MODIFF_CUDA(cudaGetDeviceProperties(&p, dev));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return MODIFF_OK;
}

int32_t modiff_out_h(const modiff_conv_geom* g) { return g ? derive(*g).ho : 0; }
int32_t modiff_out_w(const modiff_conv_geom* g) { return g ? derive(*g).wo : 0; }

int64_t modiff_codes_bytes(const modiff_conv_geom* g) {
  if (!g) return 0;
  Derived d = derive(*g);
  return (int64_t)g->batch * d.nplanes * d.hp * d.wp * d.cp;
}

int32_t modiff_wcodes_rows(const modiff_conv_geom* g, int with_sum_rows) {
  if (!g) return 0;
  if (!with_sum_rows) return round_up(g->cout, 128);
  return ceil_div(g->cout, 128) * 144;
}

int64_t modiff_wcodes_bytes(const modiff_conv_geom* g, int with_sum_rows) {
  if (!g) return 0;
  Derived d = derive(*g);
  return (int64_t)modiff_wcodes_rows(g, with_sum_rows) * d.taps * d.kp;
}

}  // extern "C"
