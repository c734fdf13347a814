// Host-side fused accumulator / optimizer math for the offload path (OpenMP outer loop, compiler
// vectorised inner loop, bf16 <-> fp32 by bit manipulation with round-to-nearest-even).
// Same six entry points as the reference's `hippo_fused_cpu` extension
// (src/training/param_offload/cpu_fused.py:109-828): add-many, zero-many, adam step, inf/nan count,
// sum of squares, scale-many. dtype codes: 0 = fp32, 1 = bf16.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <omp.h>

namespace {
inline float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f32_to_bf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040);   // quiet NaN
  u += 0x7FFFu + ((u >> 16) & 1u);                                                                 // RNE
  return (uint16_t)(u >> 16);
}
inline float ld(const void* p, int64_t i, int dt) { return dt ? bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i]; }
inline void st(void* p, int64_t i, int dt, float v) { if (dt) ((uint16_t*)p)[i] = f32_to_bf16(v); else ((float*)p)[i] = v; }
constexpr int64_t kGrain = 1 << 16;
}  // namespace

extern "C" {

// dst[i] += src[i] for n tensor pairs
void hippo_host_add_into_many(void** dst, const void** src, const int64_t* numel, const int* dst_dt, const int* src_dt, int n) {
  for (int t = 0; t < n; ++t) {
    void* d = dst[t]; const void* s = src[t]; const int dd = dst_dt[t], sd = src_dt[t]; const int64_t m = numel[t];
#pragma omp parallel for schedule(static) if (m > kGrain)
    for (int64_t b = 0; b < m; b += 4096) {
      const int64_t e = b + 4096 < m ? b + 4096 : m;
      for (int64_t i = b; i < e; ++i) st(d, i, dd, ld(d, i, dd) + ld(s, i, sd));
    }
  }
}

void hippo_host_zero_many(void** dst, const int64_t* nbytes, int n) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int t = 0; t < n; ++t) std::memset(dst[t], 0, (size_t)nbytes[t]);
}

void hippo_host_scale_many(void** dst, const int64_t* numel, const int* dt, int n, float scale) {
  for (int t = 0; t < n; ++t) {
    void* d = dst[t]; const int dd = dt[t]; const int64_t m = numel[t];
#pragma omp parallel for schedule(static) if (m > kGrain)
    for (int64_t i = 0; i < m; ++i) st(d, i, dd, ld(d, i, dd) * scale);
  }
}

double hippo_host_l2_norm_sq(const void** src, const int64_t* numel, const int* dt, int n) {
  double total = 0.0;
  for (int t = 0; t < n; ++t) {
    const void* s = src[t]; const int sd = dt[t]; const int64_t m = numel[t];
    double acc = 0.0;
#pragma omp parallel for reduction(+ : acc) schedule(static) if (m > kGrain)
    for (int64_t i = 0; i < m; ++i) { double v = ld(s, i, sd); acc += v * v; }
    total += acc;
  }
  return total;
}

int64_t hippo_host_inf_nan_count(const void** src, const int64_t* numel, const int* dt, int n) {
  int64_t total = 0;
  for (int t = 0; t < n; ++t) {
    const void* s = src[t]; const int sd = dt[t]; const int64_t m = numel[t];
    int64_t acc = 0;
#pragma omp parallel for reduction(+ : acc) schedule(static) if (m > kGrain)
    for (int64_t i = 0; i < m; ++i) acc += std::isfinite(ld(s, i, sd)) ? 0 : 1;
    total += acc;
  }
  return total;
}

// AdamW moments on the host; writes the update factor (m_hat / (sqrt(v_hat) + eps)) over the gradient buffer.
// compat != 0 reproduces the reference variant (second moment from m^2, no first-moment bias correction).
void hippo_host_adam_step(void* grad, void* m, void* v, int64_t n, int g_dt, int m_dt, int v_dt, float b1, float b2,
                          float eps, float bc1, float bc2, float gscale, int compat) {
#pragma omp parallel for schedule(static) if (n > kGrain)
  for (int64_t i = 0; i < n; ++i) {
    float g = ld(grad, i, g_dt) * gscale;
    float mv = b1 * ld(m, i, m_dt) + (1.f - b1) * g;
    float vv = b2 * ld(v, i, v_dt) + (1.f - b2) * (compat ? mv * mv : g * g);
    st(m, i, m_dt, mv); st(v, i, v_dt, vv);
    float upd = compat ? mv / (std::sqrt(vv / bc2) + eps) : (mv / bc1) / (std::sqrt(vv / bc2) + eps);
    st(grad, i, g_dt, upd);
  }
}

int hippo_host_num_threads() { return omp_get_max_threads(); }

}  // extern "C"
