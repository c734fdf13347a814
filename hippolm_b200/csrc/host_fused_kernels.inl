// Serial range kernels of the host-side fused accumulator / optimizer math. This file is included twice by
// host_fused.cpp, once under `#pragma GCC target` for AVX-512 and once for the baseline (AVX2) build, each time inside
// its own namespace; the loops are plain C++ that the compiler vectorises for the instruction set of the inclusion.
// Element types are template parameters (float or bf16 as uint16_t bits), so no loop carries a dtype branch.
// bf16 <-> fp32 by bit manipulation, narrowing with round-to-nearest-even (NaN kept quiet), all branch-free.

struct F32 { typedef float T; static inline float ld(const float* p, int64_t i) { return p[i]; }
             static inline void st(float* p, int64_t i, float v) { p[i] = v; } };
struct BF16 {
  typedef uint16_t T;
  static inline float ld(const uint16_t* p, int64_t i) {
    uint32_t u = (uint32_t)p[i] << 16; float f; __builtin_memcpy(&f, &u, 4); return f;
  }
  static inline void st(uint16_t* p, int64_t i, float v) {
    uint32_t u; __builtin_memcpy(&u, &v, 4);
    const uint32_t rne = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    const uint32_t nan = (u >> 16) | 0x0040u;
    const bool is_nan = (u & 0x7FFFFFFFu) > 0x7F800000u;
    p[i] = (uint16_t)(is_nan ? nan : rne);
  }
};

template <class D, class S>
static void add_range(void* dv, const void* sv, int64_t b, int64_t e) {
  typename D::T* __restrict__ d = (typename D::T*)dv; const typename S::T* __restrict__ s = (const typename S::T*)sv;
#pragma omp simd
  for (int64_t i = b; i < e; ++i) D::st(d, i, D::ld(d, i) + S::ld(s, i));
}

template <class D>
static void scale_range(void* dv, float scale, int64_t b, int64_t e) {
  typename D::T* __restrict__ d = (typename D::T*)dv;
#pragma omp simd
  for (int64_t i = b; i < e; ++i) D::st(d, i, D::ld(d, i) * scale);
}

template <class S>
static double sumsq_range(const void* sv, int64_t b, int64_t e) {
  const typename S::T* __restrict__ s = (const typename S::T*)sv;
  double acc = 0.0;
#pragma omp simd reduction(+ : acc)
  for (int64_t i = b; i < e; ++i) { const double v = (double)S::ld(s, i); acc += v * v; }
  return acc;
}

static int64_t nonfinite_range_f32(const void* sv, int64_t b, int64_t e) {
  const uint32_t* __restrict__ s = (const uint32_t*)sv;
  int64_t acc = 0;
#pragma omp simd reduction(+ : acc)
  for (int64_t i = b; i < e; ++i) acc += ((s[i] & 0x7F800000u) == 0x7F800000u) ? 1 : 0;   // exponent all ones: inf or NaN
  return acc;
}
static int64_t nonfinite_range_bf16(const void* sv, int64_t b, int64_t e) {
  const uint16_t* __restrict__ s = (const uint16_t*)sv;
  int64_t acc = 0;
#pragma omp simd reduction(+ : acc)
  for (int64_t i = b; i < e; ++i) acc += ((s[i] & 0x7F80u) == 0x7F80u) ? 1 : 0;
  return acc;
}

// AdamW moments; the update factor overwrites the gradient. COMPAT: second moment from m^2, no first-moment correction.
template <class G, class M, class V, bool COMPAT>
static void adam_range(void* gv, void* mv_, void* vv_, int64_t b, int64_t e, float b1, float b2, float eps, float bc1,
                       float bc2, float gscale) {
  typename G::T* __restrict__ g = (typename G::T*)gv; typename M::T* __restrict__ m = (typename M::T*)mv_;
  typename V::T* __restrict__ v = (typename V::T*)vv_;
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
#pragma omp simd
  for (int64_t i = b; i < e; ++i) {
    const float gr = G::ld(g, i) * gscale;
    const float mn = b1 * M::ld(m, i) + (1.f - b1) * gr;
    const float vn = b2 * V::ld(v, i) + (1.f - b2) * (COMPAT ? mn * mn : gr * gr);
    M::st(m, i, mn); V::st(v, i, vn);
    const float den = __builtin_sqrtf(vn * inv_bc2) + eps;
    G::st(g, i, (COMPAT ? mn : mn * inv_bc1) / den);
  }
}

static void fill_table(KernelTable& t) {
  t.add[0][0] = add_range<F32, F32>;   t.add[0][1] = add_range<F32, BF16>;
  t.add[1][0] = add_range<BF16, F32>;  t.add[1][1] = add_range<BF16, BF16>;
  t.scale[0] = scale_range<F32>;       t.scale[1] = scale_range<BF16>;
  t.sumsq[0] = sumsq_range<F32>;       t.sumsq[1] = sumsq_range<BF16>;
  t.nonfinite[0] = nonfinite_range_f32; t.nonfinite[1] = nonfinite_range_bf16;
#define HIPPO_ADAM(gi, mi, vi, G_, M_, V_) \
  t.adam[gi][mi][vi][0] = adam_range<G_, M_, V_, false>; t.adam[gi][mi][vi][1] = adam_range<G_, M_, V_, true>;
  HIPPO_ADAM(0, 0, 0, F32, F32, F32)   HIPPO_ADAM(0, 0, 1, F32, F32, BF16)
  HIPPO_ADAM(0, 1, 0, F32, BF16, F32)  HIPPO_ADAM(0, 1, 1, F32, BF16, BF16)
  HIPPO_ADAM(1, 0, 0, BF16, F32, F32)  HIPPO_ADAM(1, 0, 1, BF16, F32, BF16)
  HIPPO_ADAM(1, 1, 0, BF16, BF16, F32) HIPPO_ADAM(1, 1, 1, BF16, BF16, BF16)
#undef HIPPO_ADAM
}
