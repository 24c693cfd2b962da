// Shared device helpers for the pylo_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <type_traits>

#include "pylo_b200.h"

#define NT 256                 // threads per CTA in the streaming kernels
#define NWARP (NT / 32)
#define SUMS_LO 38             // desc.sums: [0,30) feature sums, [30,38) VeLO statistics, [38,46) their low parts
#define SUMS_STRIDE 48

// ----------------------------------------------------------------------------------------------
// family traits: feature counts and where the twelve vector-only features sit in reference order
// (learned_optimizer.cu:59-96, celo2_kernel.cu:87-124, velo_kernel.cu:123-162)
// ----------------------------------------------------------------------------------------------
template <int FAM>
struct Fam;
template <>
struct Fam<PYLO_FAM_ADAFAC> {
  static constexpr int NF = 28, NIN = 39, H = 32, NOUT = 2;
  static constexpr int R = 13, C = 16, RR = 19, RC = 22;  // fac_r, fac_c, rsqrt(fac_r), rsqrt(fac_c)
};
template <>
struct Fam<PYLO_FAM_CELO2> {
  static constexpr int NF = 30, NIN = 30, H = 8, NOUT = 3;
  static constexpr int R = 15, C = 18, RR = 21, RC = 24;
};
template <>
struct Fam<PYLO_FAM_VELO> {
  static constexpr int NF = 30, NIN = 30, H = 4, NOUT = 3;
  static constexpr int R = 15, C = 18, RR = 21, RC = 24;
};

template <int FAM>
__host__ __device__ constexpr bool is_vec_feature(int j) {
  return j >= Fam<FAM>::R && j < Fam<FAM>::R + 12;
}

// folded-network layout inside desc.wfold (floats)
template <int FAM>
struct Fold {
  using F = Fam<FAM>;
  static constexpr int W1 = 0;                    // [NF][H], k-major
  static constexpr int B1 = W1 + F::NF * F::H;    // [H]
  static constexpr int W2 = B1 + F::H;            // [H][H], k-major
  static constexpr int B2 = W2 + F::H * F::H;     // [H]
  static constexpr int W3 = B2 + F::H;            // [H][2], k-major (only direction and magnitude)
  static constexpr int B3 = W3 + F::H * 2;        // [2]
  static constexpr int SC = B3 + 2;               // [0] param_scale (VeLO), [1] lr_eff
  static constexpr int W3P = SC + 2;              // [H/2][4]: (dir[2j], dir[2j+1], mag[2j], mag[2j+1]) for packed dot products
  static constexpr int SIZE = W3P + 2 * F::H;
};
static_assert(Fold<PYLO_FAM_ADAFAC>::SIZE <= PYLO_WFOLD_STRIDE, "wfold too small");

// compile-time loop: guarantees static register indexing however large the unrolled body gets
template <int I, int N, class Fn>
__device__ __forceinline__ void static_for(Fn&& fn) {
  if constexpr (I < N) {
    fn(std::integral_constant<int, I>{});
    static_for<I + 1, N>(fn);
  }
}

// ----------------------------------------------------------------------------------------------
// scalar helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ float lerp_torch(float a, float b, float w) {
  // torch.lerp: a + w*(b-a) for |w| < 0.5, else b - (b-a)*(1-w)
  const float d = b - a;
  return (fabsf(w) < 0.5f) ? fmaf(w, d, a) : b - d * (1.0f - w);
}

__device__ __forceinline__ float safe_rsqrt(float x) { return rsqrtf(fmaxf(x, 1e-9f)); }

// rsqrt of a value known to be a positive normal number (v + eps with eps >= 1e-8): the bare
// hardware approximation (about 1.5 ulp), without the range fix-ups rsqrtf() carries
__device__ __forceinline__ float rsqrt_pos(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float grad_scale_of(const pylo_tensor_desc& d, const pylo_step_params& prm) {
  if (d.clip_norm <= 0.0f || prm.gnorm_sq == nullptr) return 1.0f;
  const float norm = sqrtf(*prm.gnorm_sq);
  const float denom = fmaxf(norm, d.clip_norm);
  return denom > 0.0f ? d.clip_norm / denom : 1.0f;
}

// g' = clamp(nan_to_num?(g * scale), +-clip); NaN passes through the clamp like torch.clamp
__device__ __forceinline__ float xform_grad(float g, float gs, float clip, int nan2num) {
  g *= gs;
  if (nan2num) {
    if (g != g) g = 0.0f;
    else if (isinf(g)) g = g > 0 ? 3.4028234663852886e38f : -3.4028234663852886e38f;
  }
  return (g != g) ? g : fminf(fmaxf(g, -clip), clip);
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// Shared-memory loads of the network weights.  They are issued as volatile PTX so that the
// compiler neither hoists thousands of loop-invariant weight loads out of the element loop
// (which would spill them to local memory) nor merges them across elements.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
template <int OFF_FLOATS>
__device__ __forceinline__ float4 lds4(uint32_t base) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(base), "n"(OFF_FLOATS * 4));
  return v;
}
template <int OFF_FLOATS>
__device__ __forceinline__ float2 lds2(uint32_t base) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(base), "n"(OFF_FLOATS * 4));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}

// Deterministic block sum of one float; result valid in every thread.  s_red: >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* s_red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) s_red[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += s_red[w];
    s_red[32] = t;
  }
  __syncthreads();
  return s_red[32];
}

// Deterministic block reduction of N per-thread accumulators; thread j < N writes out[j].
// s_red: NWARP * N floats.
template <int N>
__device__ __forceinline__ void block_reduce_store(float (&acc)[N], float* s_red, float* out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float v = warp_sum(acc[j]);
    if (lane == 0) s_red[warp * N + j] = v;
  }
  __syncthreads();
  if (threadIdx.x < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) t += s_red[w * N + threadIdx.x];
    out[threadIdx.x] = t;
  }
  __syncthreads();
}

// a / b vector indices of element idx of a [O,X,M,Y,I] tensor
struct Geo {
  uint32_t X, M, Y, I;
  __device__ __forceinline__ void split(uint64_t idx, uint64_t& a, uint64_t& b) const {
    const uint64_t i = idx % I;
    uint64_t t = idx / I;
    const uint64_t y = t % Y;
    t /= Y;
    const uint64_t m = t % M;
    t /= M;
    const uint64_t x = t % X;
    const uint64_t o = t / X;
    a = ((o * X + x) * M + m) * I + i;
    b = ((o * M + m) * Y + y) * I + i;
  }
};
