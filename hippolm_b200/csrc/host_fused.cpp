// Host-side fused accumulator / optimizer math for the offload path: OpenMP over blocks of elements, vectorised range
// kernels inside (host_fused_kernels.inl), chosen once per process by CPUID: the AVX-512 build of the kernels where the
// CPU has AVX-512 F/BW/DQ/VL, the AVX2 build otherwise (HIPPO_HOST_ISA=avx2 forces the latter).
// Same six entry points as the reference's `hippo_fused_cpu` extension
// (src/training/param_offload/cpu_fused.py:109-828): add-many, zero-many, adam step, inf/nan count,
// sum of squares, scale-many. dtype codes: 0 = fp32, 1 = bf16.
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <omp.h>

namespace {

struct KernelTable {
  void (*add[2][2])(void*, const void*, int64_t, int64_t);                       // [dst dtype][src dtype]
  void (*scale[2])(void*, float, int64_t, int64_t);
  double (*sumsq[2])(const void*, int64_t, int64_t);
  int64_t (*nonfinite[2])(const void*, int64_t, int64_t);
  void (*adam[2][2][2][2])(void*, void*, void*, int64_t, int64_t, float, float, float, float, float, float);   // [g][m][v][compat]
};

#pragma GCC push_options
#pragma GCC target("avx512f,avx512bw,avx512dq,avx512vl,fma,prefer-vector-width=512")
namespace isa_avx512 {
#include "host_fused_kernels.inl"
}
#pragma GCC pop_options

namespace isa_base {          // the instruction set of the command line (x86-64-v3: AVX2 + FMA)
#include "host_fused_kernels.inl"
}

struct Dispatch {
  KernelTable t;
  int isa;                    // 0 = AVX2 build, 1 = AVX-512 build
  Dispatch() {
    __builtin_cpu_init();
    const char* force = std::getenv("HIPPO_HOST_ISA");
    const bool want512 = !(force && std::strcmp(force, "avx2") == 0);
    const bool has512 = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
                        __builtin_cpu_supports("avx512dq") && __builtin_cpu_supports("avx512vl");
    isa = (want512 && has512) ? 1 : 0;
    if (isa) isa_avx512::fill_table(t); else isa_base::fill_table(t);
  }
};
const Dispatch& dispatch() { static const Dispatch d; return d; }

constexpr int64_t kBlock = 1 << 15;        // elements per work item of the OpenMP loops
constexpr int64_t kGrain = 1 << 16;        // below this a tensor is handled by the calling thread alone

}  // namespace

extern "C" {

// dst[i] += src[i] for n tensor pairs
void hippo_host_add_into_many(void** dst, const void** src, const int64_t* numel, const int* dst_dt, const int* src_dt, int n) {
  const KernelTable& k = dispatch().t;
  for (int t = 0; t < n; ++t) {
    void* d = dst[t]; const void* s = src[t]; const int64_t m = numel[t];
    auto fn = k.add[dst_dt[t] ? 1 : 0][src_dt[t] ? 1 : 0];
#pragma omp parallel for schedule(static) if (m > kGrain)
    for (int64_t b = 0; b < m; b += kBlock) fn(d, s, b, b + kBlock < m ? b + kBlock : m);
  }
}

void hippo_host_zero_many(void** dst, const int64_t* nbytes, int n) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int t = 0; t < n; ++t) std::memset(dst[t], 0, (size_t)nbytes[t]);
}

void hippo_host_scale_many(void** dst, const int64_t* numel, const int* dt, int n, float scale) {
  const KernelTable& k = dispatch().t;
  for (int t = 0; t < n; ++t) {
    void* d = dst[t]; const int64_t m = numel[t];
    auto fn = k.scale[dt[t] ? 1 : 0];
#pragma omp parallel for schedule(static) if (m > kGrain)
    for (int64_t b = 0; b < m; b += kBlock) fn(d, scale, b, b + kBlock < m ? b + kBlock : m);
  }
}

double hippo_host_l2_norm_sq(const void** src, const int64_t* numel, const int* dt, int n) {
  const KernelTable& k = dispatch().t;
  double total = 0.0;
  for (int t = 0; t < n; ++t) {
    const void* s = src[t]; const int64_t m = numel[t];
    auto fn = k.sumsq[dt[t] ? 1 : 0];
    double acc = 0.0;
#pragma omp parallel for reduction(+ : acc) schedule(static) if (m > kGrain)
    for (int64_t b = 0; b < m; b += kBlock) acc += fn(s, b, b + kBlock < m ? b + kBlock : m);
    total += acc;
  }
  return total;
}

int64_t hippo_host_inf_nan_count(const void** src, const int64_t* numel, const int* dt, int n) {
  const KernelTable& k = dispatch().t;
  int64_t total = 0;
  for (int t = 0; t < n; ++t) {
    const void* s = src[t]; const int64_t m = numel[t];
    auto fn = k.nonfinite[dt[t] ? 1 : 0];
    int64_t acc = 0;
#pragma omp parallel for reduction(+ : acc) schedule(static) if (m > kGrain)
    for (int64_t b = 0; b < m; b += kBlock) acc += fn(s, b, b + kBlock < m ? b + kBlock : m);
    total += acc;
  }
  return total;
}

// AdamW moments on the host; writes the update factor (m_hat / (sqrt(v_hat) + eps)) over the gradient buffer.
// compat != 0 reproduces the reference variant (second moment from m^2, no first-moment bias correction).
void hippo_host_adam_step(void* grad, void* m, void* v, int64_t n, int g_dt, int m_dt, int v_dt, float b1, float b2,
                          float eps, float bc1, float bc2, float gscale, int compat) {
  auto fn = dispatch().t.adam[g_dt ? 1 : 0][m_dt ? 1 : 0][v_dt ? 1 : 0][compat ? 1 : 0];
#pragma omp parallel for schedule(static) if (n > kGrain)
  for (int64_t b = 0; b < n; b += kBlock) fn(grad, m, v, b, b + kBlock < n ? b + kBlock : n, b1, b2, eps, bc1, bc2, gscale);
}

int hippo_host_num_threads() { return omp_get_max_threads(); }

// 1 = the AVX-512 build of the kernels is in use, 0 = the AVX2 build
int hippo_host_isa() { return dispatch().isa; }

}  // extern "C"
