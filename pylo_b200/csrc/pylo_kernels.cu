// pylo_b200: learned-optimizer step kernels for B200 (sm_100a) and their C ABI.
//
// One optimizer step is a fixed sequence of launches over a device-resident
// table of tensor descriptors and tile lists (see include/pylo_b200.h):
//   [grad_sumsq] -> rowcol_sums (A) -> factor_update (A2) -> state_moments (B)
//   -> finalize_moments (B2) -> [velo front end] -> prep_apply (P) -> apply (C)
//   -> [celo2 post] / [adamw]
// All reductions go through fixed-slot partials and fixed-order final sums, so
// results are bit-reproducible from run to run (no floating-point atomics).

#include <string.h>

#include <mutex>

#include "pylo_common.cuh"

// ================================================================================================
// feature construction (reference order; learned_optimizer.cu:59-96, celo2_kernel.cu:87-124)
// ================================================================================================
template <int FAM>
__device__ __forceinline__ void elem_features(float* f, float g, float p, float m0, float m1, float m2, float v,
                                              float rs, float k0, float k1, float k2) {
  if (FAM == PYLO_FAM_ADAFAC) {
    f[0] = g; f[1] = p; f[2] = m0; f[3] = m1; f[4] = m2; f[5] = v;
    f[6] = m0 * rs; f[7] = m1 * rs; f[8] = m2 * rs; f[9] = rs;
    f[10] = k0 * g; f[11] = k1 * g; f[12] = k2 * g;
    f[25] = k0 * m0; f[26] = k1 * m1; f[27] = k2 * m2;
  } else {
    f[0] = g; f[1] = fminf(fmaxf(g, -0.1f), 0.1f); f[2] = p; f[3] = m0; f[4] = m1; f[5] = m2; f[6] = v;
    f[7] = m0 * rs; f[8] = m1 * rs; f[9] = m2 * rs; f[10] = rs;
    f[11] = k0 * g; f[12] = k1 * g; f[13] = k2 * g; f[14] = g * rs;
    f[27] = k0 * m0; f[28] = k1 * m1; f[29] = k2 * m2;
  }
}

template <int FAM>
__device__ __forceinline__ void vec_features(float* f, float r0, float r1, float r2, float c0, float c1, float c2) {
  using F = Fam<FAM>;
  f[F::R] = r0; f[F::R + 1] = r1; f[F::R + 2] = r2;
  f[F::C] = c0; f[F::C + 1] = c1; f[F::C + 2] = c2;
  f[F::RR] = rsqrtf(r0 + 1e-8f); f[F::RR + 1] = rsqrtf(r1 + 1e-8f); f[F::RR + 2] = rsqrtf(r2 + 1e-8f);
  f[F::RC] = rsqrtf(c0 + 1e-8f); f[F::RC + 1] = rsqrtf(c1 + 1e-8f); f[F::RC + 2] = rsqrtf(c2 + 1e-8f);
}

// ================================================================================================
// global gradient norm
// ================================================================================================
__global__ void __launch_bounds__(NT) k_grad_sumsq(const pylo_gvec* __restrict__ descs,
                                                   const pylo_tile* __restrict__ tiles, int n_tiles,
                                                   float* __restrict__ scratch) {
  __shared__ float s_red[40];
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const pylo_tile tl = tiles[t];
    const float* g = descs[tl.tensor].g + tl.start;
    const int64_t rem = descs[tl.tensor].n - tl.start;
    const int cnt = rem < PYLO_TILE_ELEMS ? (int)rem : PYLO_TILE_ELEMS;
    float acc = 0.f;
    if ((((uintptr_t)g) & 15) == 0) {
      const int c4 = cnt & ~3;
      for (int i = threadIdx.x * 4; i < c4; i += NT * 4) {
        const float4 q = ldg4(g + i);
        acc += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
      }
      for (int i = c4 + threadIdx.x; i < cnt; i += NT) acc += g[i] * g[i];
    } else {
      for (int i = threadIdx.x; i < cnt; i += NT) acc += g[i] * g[i];
    }
    const float tot = block_sum(acc, s_red);
    if (threadIdx.x == 0) scratch[t] = tot;
  }
}

__global__ void __launch_bounds__(1024) k_sum_final(const float* __restrict__ scratch, int n, float* __restrict__ out) {
  __shared__ double s_d[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += (double)scratch[i];
  acc = warp_sum_d(acc);
  if ((threadIdx.x & 31) == 0) s_d[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_d[w];
    out[0] = (float)t;
  }
}

// ================================================================================================
// Phase A: row / column sums of g'^2 + 1e-30
// ================================================================================================
__global__ void __launch_bounds__(NT) k_rowcol_fast(const pylo_tensor_desc* __restrict__ descs,
                                                    const pylo_atile* __restrict__ atiles, int n_atiles,
                                                    const pylo_step_params prm) {
  __shared__ float s_col[NWARP][PYLO_A_COLS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = blockIdx.x; t < n_atiles; t += gridDim.x) {
    const pylo_atile at = atiles[t];
    const pylo_tensor_desc& d = descs[at.tensor];
    const int X = d.X, Y = d.Y, rb = d.rb;
    const int row0 = at.strip * rb;
    const int rows = min(rb, X - row0);
    const int col0 = at.cb * PYLO_A_COLS;
    const float gs = grad_scale_of(d, prm);
    float colacc[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) colacc[j] = 0.f;
    for (int r = warp; r < rows; r += NWARP) {
      const int x = row0 + r;
      const float* grow = d.g + (int64_t)x * Y + col0;
      float rowsum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = lane * 4 + j * 128;
        if (col0 + c < Y) {
          const float4 q = ldg4(grow + c);
          const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float g = xform_grad(e[u], gs, prm.clip_val, prm.nan_to_num);
            const float s = g * g + 1e-30f;
            colacc[j * 4 + u] += s;
            rowsum += s;
          }
        }
      }
      rowsum = warp_sum(rowsum);
      if (lane == 0) d.part_a[(int64_t)x * d.n_cb + at.cb] = rowsum;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) st4(&s_col[warp][lane * 4 + j * 128], make_float4(colacc[j * 4], colacc[j * 4 + 1], colacc[j * 4 + 2], colacc[j * 4 + 3]));
    __syncthreads();
    {
      const int c = threadIdx.x * 4;
      if (col0 + c < Y) {
        float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < NWARP; ++w) {
          const float4 q = ld4(&s_col[w][c]);
          tot.x += q.x; tot.y += q.y; tot.z += q.z; tot.w += q.w;
        }
        st4(d.part_b + (int64_t)at.strip * Y + col0 + c, tot);
      }
    }
    __syncthreads();
  }
}

// Second level of the column sums: sum_b[y] = sum over strips of part_b[strip][y], strips in order.
// One work item = 1024 columns of one tensor; a thread owns a float4 of columns.
__global__ void __launch_bounds__(NT) k_colpart_reduce(const pylo_tensor_desc* __restrict__ descs,
                                                       const pylo_atile* __restrict__ rtiles, int n_rtiles) {
  for (int t = blockIdx.x; t < n_rtiles; t += gridDim.x) {
    const pylo_atile rt = rtiles[t];
    const pylo_tensor_desc& d = descs[rt.tensor];
    const int Y = d.Y, strips = d.n_strips;
    const int y = rt.cb * PYLO_A_COLS + threadIdx.x * 4;
    if (y >= Y) continue;
    const float* __restrict__ src = d.part_b + y;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int r = 0;
    for (; r + 4 <= strips; r += 4) {  // four loads in flight, added in strip order
      const float4 q0 = ld4(src + (int64_t)r * Y), q1 = ld4(src + (int64_t)(r + 1) * Y);
      const float4 q2 = ld4(src + (int64_t)(r + 2) * Y), q3 = ld4(src + (int64_t)(r + 3) * Y);
      acc.x = (((acc.x + q0.x) + q1.x) + q2.x) + q3.x; acc.y = (((acc.y + q0.y) + q1.y) + q2.y) + q3.y;
      acc.z = (((acc.z + q0.z) + q1.z) + q2.z) + q3.z; acc.w = (((acc.w + q0.w) + q1.w) + q2.w) + q3.w;
    }
    for (; r < strips; ++r) {
      const float4 q = ld4(src + (int64_t)r * Y);
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    st4(d.sum_b + y, acc);
  }
}

// GENERIC tensors: one warp per output vector element, lanes stride over the reduced axis.
__global__ void __launch_bounds__(NT) k_rowcol_generic(const pylo_tensor_desc* __restrict__ descs,
                                                       const int32_t* __restrict__ ids, int slices,
                                                       const pylo_step_params prm) {
  const pylo_tensor_desc& d = descs[ids[blockIdx.x / slices]];
  const int slice = blockIdx.x % slices;
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t)slice * NWARP + (threadIdx.x >> 5);
  const int64_t nw = (int64_t)slices * NWARP;
  const int64_t X = d.X, M = d.M, Y = d.Y, I = d.I;
  const int64_t La = d.La, Lb = d.Lb;
  const float gs = grad_scale_of(d, prm);
  for (int64_t o = wid; o < La + Lb; o += nw) {
    float acc = 0.f;
    if (o < La) {  // a = ((o*X + x)*M + m)*I + i ; sum over y
      const int64_t i = o % I, omx = o / I;
      const int64_t base = omx * Y * I + i;
      for (int64_t y = lane; y < Y; y += 32) {
        const float g = xform_grad(d.g[base + y * I], gs, prm.clip_val, prm.nan_to_num);
        acc += g * g + 1e-30f;
      }
      acc = warp_sum(acc);
      if (lane == 0) d.sum_a[o] = acc;
    } else {  // b = ((o*M + m)*Y + y)*I + i ; sum over x
      const int64_t b = o - La;
      const int64_t i = b % I;
      int64_t t = b / I;
      const int64_t y = t % Y;
      t /= Y;
      const int64_t m = t % M, oo = t / M;
      for (int64_t x = lane; x < X; x += 32) {
        const int64_t idx = ((((oo * X + x) * M + m) * Y + y) * I) + i;
        const float g = xform_grad(d.g[idx], gs, prm.clip_val, prm.nan_to_num);
        acc += g * g + 1e-30f;
      }
      acc = warp_sum(acc);
      if (lane == 0) d.sum_b[b] = acc;
    }
  }
}

// ================================================================================================
// Phase A2: factored accumulators, factors, closed-form vector-feature moments.  One CTA per tensor.
// ================================================================================================
#define A2_NT 1024
template <int FAM>
__global__ void __launch_bounds__(A2_NT) k_factor_update(const pylo_tensor_desc* __restrict__ descs,
                                                         const pylo_step_params prm) {
  using F = Fam<FAM>;
  __shared__ float s_red[40];
  __shared__ float s_mean[8];
  const pylo_tensor_desc& d = descs[blockIdx.x];
  const int tid = threadIdx.x;
  if (tid < PYLO_STAT_STRIDE) d.closed[tid] = 0.f;
  if (d.mode == PYLO_MODE_VEC1D) return;
  const int64_t X = d.X, Y = d.Y;
  const int64_t La = d.La, Lb = d.Lb;

  // 1. finish the row/column sums of the float4 path
  if (d.mode == PYLO_MODE_FAST2D) {
    for (int64_t x = tid; x < X; x += A2_NT) {
      float s = 0.f;
      for (int c = 0; c < d.n_cb; ++c) s += d.part_a[x * d.n_cb + c];
      d.sum_a[x] = s;
    }
    // the column sums were finished by k_colpart_reduce
  }
  __syncthreads();

  // 2. EMA of the two accumulators: lerp(acc, mean, 1 - beta_fac[k])
  for (int64_t i = tid; i < La; i += A2_NT) {
    const float mean = d.sum_a[i] / (float)Y;
#pragma unroll
    for (int k = 0; k < 3; ++k) d.fac_a[k * La + i] = lerp_torch(d.fac_a[k * La + i], mean, prm.w_f[k]);
  }
  for (int64_t i = tid; i < Lb; i += A2_NT) {
    const float mean = d.sum_b[i] / (float)X;
#pragma unroll
    for (int k = 0; k < 3; ++k) d.fac_b[k * Lb + i] = lerp_torch(d.fac_b[k * Lb + i], mean, prm.w_f[k]);
  }
  __syncthreads();

  // 3. row_factor = safe_rsqrt(fac_r / (mean over the reduce axis + 1e-9)), col_factor = safe_rsqrt(fac_c)
  const float* fac_r = d.r_is_a ? d.fac_a : d.fac_b;
  const float* fac_c = d.r_is_a ? d.fac_b : d.fac_a;
  float* f_r = d.r_is_a ? d.f_a : d.f_b;
  float* f_c = d.r_is_a ? d.f_b : d.f_a;
  const int64_t Lr = d.r_is_a ? La : Lb, Lc = d.r_is_a ? Lb : La;
  const int64_t pre = d.rcm_pre, A = d.rcm_A, post = d.rcm_post;
  if (post == 1 && pre <= 8) {
    for (int pr = 0; pr < pre; ++pr) {
      float acc = 0.f;
      for (int64_t a = tid; a < A; a += A2_NT) acc += fac_r[pr * A + a];
      const float tot = block_sum(acc, s_red);
      if (tid == 0) s_mean[pr] = tot / (float)A;
    }
    __syncthreads();
    for (int64_t e = tid; e < 3 * Lr; e += A2_NT) f_r[e] = safe_rsqrt(fac_r[e] / (s_mean[e / A] + 1e-9f));
  } else if (post == 1) {
    const int lane = tid & 31;
    for (int64_t pr = tid >> 5; pr < pre; pr += A2_NT / 32) {
      float acc = 0.f;
      for (int64_t a = lane; a < A; a += 32) acc += fac_r[pr * A + a];
      acc = warp_sum(acc);
      acc = __shfl_sync(0xffffffffu, acc, 0) / (float)A;
      for (int64_t a = lane; a < A; a += 32) f_r[pr * A + a] = safe_rsqrt(fac_r[pr * A + a] / (acc + 1e-9f));
    }
  } else {
    for (int64_t o = tid; o < pre * post; o += A2_NT) {
      const int64_t pr = o / post, po = o % post;
      float acc = 0.f;
      for (int64_t a = 0; a < A; ++a) acc += fac_r[(pr * A + a) * post + po];
      acc /= (float)A;
      for (int64_t a = 0; a < A; ++a) {
        const int64_t e = (pr * A + a) * post + po;
        f_r[e] = safe_rsqrt(fac_r[e] / (acc + 1e-9f));
      }
    }
  }
  for (int64_t e = tid; e < 3 * Lc; e += A2_NT) f_c[e] = safe_rsqrt(fac_c[e]);
  __syncthreads();

  // 4. "a" factors interleaved per index for the float4 path
  if (d.mode == PYLO_MODE_FAST2D) {
    for (int64_t i = tid; i < La; i += A2_NT)
      st4(d.fx + 4 * i, make_float4(d.f_a[i], d.f_a[La + i], d.f_a[2 * La + i], 0.f));
  }

  // 5. closed-form sums of squares of the features that depend on one vector only: every
  //    vector entry is seen by n / L elements of the tensor.
  {
    const float mult_r = (float)(d.n / Lr), mult_c = (float)(d.n / Lc);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      float s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f;
      for (int64_t i = tid; i < Lr; i += A2_NT) {
        const float r = fac_r[k * Lr + i];
        s1 += r * r;
        const float q = rsqrtf(r + 1e-8f);
        s2 += q * q;
      }
      for (int64_t i = tid; i < Lc; i += A2_NT) {
        const float c = fac_c[k * Lc + i];
        s3 += c * c;
        const float q = rsqrtf(c + 1e-8f);
        s4 += q * q;
      }
      s1 = block_sum(s1, s_red);
      s2 = block_sum(s2, s_red);
      s3 = block_sum(s3, s_red);
      s4 = block_sum(s4, s_red);
      if (tid == 0) {
        d.closed[F::R + k] = s1 * mult_r;
        d.closed[F::RR + k] = s2 * mult_r;
        d.closed[F::C + k] = s3 * mult_c;
        d.closed[F::RC + k] = s4 * mult_c;
      }
    }
  }
}

// ================================================================================================
// Phase B: state update + per-tile sums of squares of the element-wise features
// ================================================================================================
template <int FAM>
struct BAcc {
  static constexpr int N = Fam<FAM>::NF + (FAM == PYLO_FAM_VELO ? 8 : 0);
};

template <int FAM, bool VECF>
__device__ __forceinline__ void accumulate(float (&acc)[BAcc<FAM>::N], const float* f) {
#pragma unroll
  for (int j = 0; j < Fam<FAM>::NF; ++j) {
    if (!VECF && is_vec_feature<FAM>(j)) continue;
    acc[j] = fmaf(f[j], f[j], acc[j]);
  }
}

template <int FAM>
__device__ __forceinline__ void velo_stats(float (&acc)[BAcc<FAM>::N], float m0, float m1, float m2, float v) {
  if (FAM == PYLO_FAM_VELO) {
    constexpr int B = Fam<FAM>::NF;
    acc[B + 0] += m0; acc[B + 1] += m1; acc[B + 2] += m2;
    acc[B + 3] = fmaf(m0, m0, acc[B + 3]); acc[B + 4] = fmaf(m1, m1, acc[B + 4]); acc[B + 5] = fmaf(m2, m2, acc[B + 5]);
    acc[B + 6] += v; acc[B + 7] = fmaf(v, v, acc[B + 7]);
  }
}

template <int FAM>
__global__ void __launch_bounds__(NT) k_state_moments(const pylo_tensor_desc* __restrict__ descs,
                                                      const pylo_tile* __restrict__ tiles, int n_tiles, int reverse,
                                                      const pylo_step_params prm) {
  using F = Fam<FAM>;
  constexpr int NACC = BAcc<FAM>::N;
  __shared__ float s_red[NWARP * NACC];
  const int tid = threadIdx.x;
  for (int tt = blockIdx.x; tt < n_tiles; tt += gridDim.x) {
    const int t = reverse ? (n_tiles - 1 - tt) : tt;
    const pylo_tile tl = tiles[t];
    const pylo_tensor_desc& d = descs[tl.tensor];
    const int64_t n = d.n, start = tl.start;
    const int cnt = (int)min((int64_t)PYLO_TILE_ELEMS, n - start);
    const float gs = grad_scale_of(d, prm);
    float acc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; ++j) acc[j] = 0.f;
    float* m0p = d.m + start;
    float* m1p = d.m + d.m_stride + start;
    float* m2p = d.m + 2 * d.m_stride + start;
    float* vp = d.v + start;
    const float* gp = d.g + start;
    const float* pp = d.p + start;

    if (d.mode == PYLO_MODE_FAST2D) {
      const uint32_t Y = d.Y;
      const bool small = n < (1ll << 32);
      for (int i = tid * 4; i < cnt; i += NT * 4) {
        const int64_t idx = start + i;
        uint32_t x, y;
        if (small) { x = (uint32_t)idx / Y; y = (uint32_t)idx - x * Y; }
        else { x = (uint32_t)(idx / Y); y = (uint32_t)(idx - (int64_t)x * Y); }
        const float4 g4 = ldg4(gp + i), p4 = ld4(pp + i);
        float4 a0 = ld4(m0p + i), a1 = ld4(m1p + i), a2 = ld4(m2p + i), v4 = ld4(vp + i);
        const float4 fa = ld4(d.fx + 4 * (int64_t)x);
        const float4 b0 = ld4(d.f_b + y), b1 = ld4(d.f_b + Y + y), b2 = ld4(d.f_b + 2 * (int64_t)Y + y);
        float ge[4] = {g4.x, g4.y, g4.z, g4.w}, pe[4] = {p4.x, p4.y, p4.z, p4.w};
        float m0e[4] = {a0.x, a0.y, a0.z, a0.w}, m1e[4] = {a1.x, a1.y, a1.z, a1.w}, m2e[4] = {a2.x, a2.y, a2.z, a2.w};
        float ve[4] = {v4.x, v4.y, v4.z, v4.w};
        const float b0e[4] = {b0.x, b0.y, b0.z, b0.w}, b1e[4] = {b1.x, b1.y, b1.z, b1.w}, b2e[4] = {b2.x, b2.y, b2.z, b2.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float g = xform_grad(ge[u], gs, prm.clip_val, prm.nan_to_num);
          velo_stats<FAM>(acc, m0e[u], m1e[u], m2e[u], ve[u]);
          m0e[u] = lerp_torch(m0e[u], g, prm.w_m[0]);
          m1e[u] = lerp_torch(m1e[u], g, prm.w_m[1]);
          m2e[u] = lerp_torch(m2e[u], g, prm.w_m[2]);
          ve[u] = lerp_torch(ve[u], g * g + prm.eps_v, prm.w_v);
          const float rs = rsqrtf(ve[u] + prm.eps_feat);
          float f[F::NF];
          elem_features<FAM>(f, g, pe[u], m0e[u], m1e[u], m2e[u], ve[u], rs, fa.x * b0e[u], fa.y * b1e[u], fa.z * b2e[u]);
          accumulate<FAM, false>(acc, f);
        }
        st4(m0p + i, make_float4(m0e[0], m0e[1], m0e[2], m0e[3]));
        st4(m1p + i, make_float4(m1e[0], m1e[1], m1e[2], m1e[3]));
        st4(m2p + i, make_float4(m2e[0], m2e[1], m2e[2], m2e[3]));
        st4(vp + i, make_float4(ve[0], ve[1], ve[2], ve[3]));
      }
    } else if (d.mode == PYLO_MODE_GENERIC) {
      const Geo geo{(uint32_t)d.X, (uint32_t)d.M, (uint32_t)d.Y, (uint32_t)d.I};
      const int64_t La = d.La, Lb = d.Lb;
      const bool vecf = d.vec_elementwise != 0;
      const float* fac_r = d.r_is_a ? d.fac_a : d.fac_b;
      const float* fac_c = d.r_is_a ? d.fac_b : d.fac_a;
      for (int i = tid; i < cnt; i += NT) {
        uint64_t a, b;
        geo.split((uint64_t)(d.idx0 + start + i), a, b);
        const float g = xform_grad(gp[i], gs, prm.clip_val, prm.nan_to_num);
        float m0 = m0p[i], m1 = m1p[i], m2 = m2p[i], v = vp[i];
        velo_stats<FAM>(acc, m0, m1, m2, v);
        m0 = lerp_torch(m0, g, prm.w_m[0]);
        m1 = lerp_torch(m1, g, prm.w_m[1]);
        m2 = lerp_torch(m2, g, prm.w_m[2]);
        v = lerp_torch(v, g * g + prm.eps_v, prm.w_v);
        m0p[i] = m0; m1p[i] = m1; m2p[i] = m2; vp[i] = v;
        const float rs = rsqrtf(v + prm.eps_feat);
        float f[F::NF];
        elem_features<FAM>(f, g, pp[i], m0, m1, m2, v, rs, d.f_a[a] * d.f_b[b], d.f_a[La + a] * d.f_b[Lb + b],
                           d.f_a[2 * La + a] * d.f_b[2 * Lb + b]);
        if (vecf) {
          const uint64_t ir = d.r_is_a ? a : b, ic = d.r_is_a ? b : a;
          const int64_t Lr = d.r_is_a ? La : Lb, Lc = d.r_is_a ? Lb : La;
          vec_features<FAM>(f, fac_r[ir], fac_r[Lr + ir], fac_r[2 * Lr + ir], fac_c[ic], fac_c[Lc + ic], fac_c[2 * Lc + ic]);
          accumulate<FAM, true>(acc, f);
        } else {
          accumulate<FAM, false>(acc, f);
        }
      }
    } else {  // VEC1D: full-size accumulators updated element-wise (AdafacLO_cuda.py:349-360, velo_cuda.py:543-546)
      float* ra = d.fac_a + start;
      float* rb = d.fac_b ? d.fac_b + start : nullptr;
      for (int i = tid; i < cnt; i += NT) {
        const float g = xform_grad(gp[i], gs, prm.clip_val, prm.nan_to_num);
        float m0 = m0p[i], m1 = m1p[i], m2 = m2p[i], v = vp[i];
        velo_stats<FAM>(acc, m0, m1, m2, v);
        m0 = lerp_torch(m0, g, prm.w_m[0]);
        m1 = lerp_torch(m1, g, prm.w_m[1]);
        m2 = lerp_torch(m2, g, prm.w_m[2]);
        v = lerp_torch(v, g * g + prm.eps_v, prm.w_v);
        m0p[i] = m0; m1p[i] = m1; m2p[i] = m2; vp[i] = v;
        const float gsq = g * g + 1e-30f;
        float r[3], c[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
          r[k] = lerp_torch(ra[k * n + i], gsq, prm.w_f[k]);
          ra[k * n + i] = r[k];
          if (rb) { c[k] = lerp_torch(rb[k * n + i], gsq, prm.w_f[k]); rb[k * n + i] = c[k]; }
          else c[k] = r[k];
        }
        const float rs = rsqrtf(v + prm.eps_feat);
        float f[F::NF];
        elem_features<FAM>(f, g, pp[i], m0, m1, m2, v, rs, safe_rsqrt(r[0] + 1e-9f), safe_rsqrt(r[1] + 1e-9f),
                           safe_rsqrt(r[2] + 1e-9f));
        vec_features<FAM>(f, r[0], r[1], r[2], c[0], c[1], c[2]);
        accumulate<FAM, true>(acc, f);
      }
    }
    float* out = d.tile_part + (int64_t)(t - d.tile0) * PYLO_STAT_STRIDE;
    block_reduce_store<NACC>(acc, s_red, out);
    if (tid >= NACC && tid < PYLO_STAT_STRIDE) out[tid] = 0.f;
  }
}

// ================================================================================================
// Phase B2: per-tensor fixed-order reduction of the tile partials
// ================================================================================================
__global__ void __launch_bounds__(NT) k_finalize_moments(const pylo_tensor_desc* __restrict__ descs) {
  __shared__ double s_d[4][64];
  const pylo_tensor_desc& d = descs[blockIdx.x];
  const int j = threadIdx.x & 63, sub = threadIdx.x >> 6;  // 4 sub-sequences of tiles x 64 columns
  double acc = 0.0;
  if (j < PYLO_STAT_STRIDE)
    for (int t = sub; t < d.n_tiles; t += 4) acc += (double)d.tile_part[(int64_t)t * PYLO_STAT_STRIDE + j];
  s_d[sub][j] = acc;
  __syncthreads();
  if (threadIdx.x < PYLO_STAT_STRIDE) {
    const double tot = ((s_d[0][j] + s_d[1][j]) + s_d[2][j]) + s_d[3][j] + (double)d.closed[j];
    const float hi = (float)tot;
    d.sums[j] = hi;
    if (j >= 30 && j < 38) d.sums[SUMS_LO + (j - 30)] = (float)(tot - (double)hi);
  }
}

// ================================================================================================
// Phase P: fold normalisers (and time features) into the first layer; tabulate vector-feature terms
// ================================================================================================
__device__ __forceinline__ float w1_at(int fam, const float* w, int j, int k) {
  // first-layer weight for hidden unit j and input k in the family's own storage order
  if (fam == PYLO_FAM_ADAFAC) return w[j * 39 + k];
  if (fam == PYLO_FAM_CELO2) return w[k * 8 + j];
  return w[j * 30 + k];
}

template <int FAM>
__global__ void __launch_bounds__(NT) k_prep_apply(const pylo_tensor_desc* __restrict__ descs,
                                                   const pylo_step_params prm) {
  using F = Fam<FAM>;
  using L = Fold<FAM>;
  constexpr int H = F::H, NF = F::NF, NIN = F::NIN;
  __shared__ float s_scale[NF];
  __shared__ float s_w1[NF * H];
  __shared__ float s_b1[H];
  const pylo_tensor_desc& d = descs[blockIdx.x];
  const int tid = threadIdx.x, slice = blockIdx.y, slices = gridDim.y;
  const float* w = d.w;
  // source offsets in the family layout
  const int o_b1 = NIN * H, o_w2 = o_b1 + H, o_b2 = o_w2 + H * H, o_w3 = o_b2 + H, o_b3 = o_w3 + H * F::NOUT;
  if (tid < NF) s_scale[tid] = rsqrtf(d.sums[tid] / (float)d.n + prm.eps_norm);
  __syncthreads();
  for (int e = tid; e < NF * H; e += NT) {
    const int k = e / H, j = e % H;
    s_w1[e] = w1_at(FAM, w, j, k) * s_scale[k];
  }
  if (tid < H) {
    float b = w[o_b1 + tid];
    if (FAM == PYLO_FAM_ADAFAC) {
      const float tau[11] = {1.f, 3.f, 10.f, 30.f, 100.f, 300.f, 1000.f, 3000.f, 10000.f, 30000.f, 100000.f};
#pragma unroll
      for (int t = 0; t < 11; ++t) b = fmaf(w1_at(FAM, w, tid, 28 + t), tanhf((d.step + prm.step_delta) / tau[t] - 1.0f), b);
    }
    s_b1[tid] = b;
  }
  __syncthreads();
  if (slice == 0) {
    float* o = d.wfold;
    for (int e = tid; e < NF * H; e += NT) o[L::W1 + e] = s_w1[e];
    if (tid < H) o[L::B1 + tid] = s_b1[tid];
    for (int e = tid; e < H * H; e += NT) {
      const int k = e / H, j = e % H;
      o[L::W2 + e] = (FAM == PYLO_FAM_CELO2) ? w[o_w2 + k * H + j] : w[o_w2 + j * H + k];
    }
    if (tid < H) o[L::B2 + tid] = w[o_b2 + tid];
    for (int e = tid; e < H * 2; e += NT) {
      const int k = e / 2, q = e % 2;
      o[L::W3 + e] = (FAM == PYLO_FAM_CELO2) ? w[o_w3 + k * F::NOUT + q] : w[o_w3 + q * H + k];
    }
    if (tid < 2) o[L::B3 + tid] = w[o_b3 + tid];
    for (int e = tid; e < H * 2; e += NT) {  // pair-major copy of the output layer
      const int jp = e / 4, r = e % 4, k = 2 * jp + (r & 1), q = r >> 1;
      o[L::W3P + e] = (FAM == PYLO_FAM_CELO2) ? w[o_w3 + k * F::NOUT + q] : w[o_w3 + q * H + k];
    }
    if (tid == 0) {
      // VeLO: param_scale = sqrt(mean(p^2) + 1e-9) from the p feature's sum (velo_kernel.cu:297)
      o[L::SC + 0] = (FAM == PYLO_FAM_VELO) ? sqrtf(d.sums[2] / (float)d.n + 1e-9f) : 1.0f;
      o[L::SC + 1] = d.lr_mult ? d.lr * d.lr_mult[0] : d.lr;
    }
  }
  if (d.mode != PYLO_MODE_FAST2D || prm.no_tables == 1) return;
  // first-layer contribution of the features that depend only on the "a" index (plus bias) / "b" index
  const int64_t La = d.X, Lb = d.Y;
  const int ka = d.r_is_a ? F::R : F::C, kra = d.r_is_a ? F::RR : F::RC;
  const int kb = d.r_is_a ? F::C : F::R, krb = d.r_is_a ? F::RC : F::RR;
  for (int64_t e = (int64_t)slice * NT + tid; e < La * H; e += (int64_t)slices * NT) {
    const int64_t i = e / H;
    const int j = (int)(e % H);
    float acc = s_b1[j];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const float r = d.fac_a[k * La + i];
      acc = fmaf(s_w1[(ka + k) * H + j], r, acc);
      acc = fmaf(s_w1[(kra + k) * H + j], rsqrtf(r + 1e-8f), acc);
    }
    if (FAM == PYLO_FAM_ADAFAC) d.h_a[e] = acc;
    else { d.h_a[2 * e] = acc; d.h_a[2 * e + 1] = acc; }  // stored as (v, v) pairs for the packed kernel
  }
  if (prm.no_tables == 2) return;  // the per-row table only
  for (int64_t e = (int64_t)slice * NT + tid; e < Lb * H; e += (int64_t)slices * NT) {
    const int64_t i = e / H;
    const int j = (int)(e % H);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const float r = d.fac_b[k * Lb + i];
      acc = fmaf(s_w1[(kb + k) * H + j], r, acc);
      acc = fmaf(s_w1[(krb + k) * H + j], rsqrtf(r + 1e-8f), acc);
    }
    d.h_b[(int64_t)j * Lb + i] = acc;  // transposed, [H][Y]: a thread reads its columns' terms with one float4
  }
}

// ================================================================================================
// Phase C: features -> network -> parameter / raw step
// ================================================================================================
// Network on E elements at once (weights are read from shared memory once per E elements).
// h1 comes in holding the bias (and, on the float4 path, the tabulated vector-feature terms);
// f holds the features in reference order.
template <int FAM, bool VECF, int E>
__device__ __forceinline__ void network(const uint32_t s_w, float (&h1)[E][Fam<FAM>::H],
                                        const float (&f)[E][Fam<FAM>::NF], float (&o0)[E], float (&o1)[E]) {
  using F = Fam<FAM>;
  using L = Fold<FAM>;
  constexpr int H = F::H;
  static_for<0, F::NF>([&](auto kc) {
    constexpr int k = decltype(kc)::value;
    if constexpr (VECF || !is_vec_feature<FAM>(k)) {
      static_for<0, H / 4>([&](auto jc) {
        constexpr int j = decltype(jc)::value * 4;
        const float4 w = lds4<L::W1 + k * H + j>(s_w);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float fk = f[e][k];
          h1[e][j] = fmaf(w.x, fk, h1[e][j]); h1[e][j + 1] = fmaf(w.y, fk, h1[e][j + 1]);
          h1[e][j + 2] = fmaf(w.z, fk, h1[e][j + 2]); h1[e][j + 3] = fmaf(w.w, fk, h1[e][j + 3]);
        }
      });
    }
  });
  float h2[E][H];
  static_for<0, H / 4>([&](auto jc) {
    constexpr int j = decltype(jc)::value * 4;
    const float4 b = lds4<L::B2 + j>(s_w);
#pragma unroll
    for (int e = 0; e < E; ++e) { h2[e][j] = b.x; h2[e][j + 1] = b.y; h2[e][j + 2] = b.z; h2[e][j + 3] = b.w; }
  });
  static_for<0, H>([&](auto kc) {
    constexpr int k = decltype(kc)::value;
    float hk[E];
#pragma unroll
    for (int e = 0; e < E; ++e) hk[e] = fmaxf(h1[e][k], 0.f);
    static_for<0, H / 4>([&](auto jc) {
      constexpr int j = decltype(jc)::value * 4;
      const float4 w = lds4<L::W2 + k * H + j>(s_w);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        h2[e][j] = fmaf(w.x, hk[e], h2[e][j]); h2[e][j + 1] = fmaf(w.y, hk[e], h2[e][j + 1]);
        h2[e][j + 2] = fmaf(w.z, hk[e], h2[e][j + 2]); h2[e][j + 3] = fmaf(w.w, hk[e], h2[e][j + 3]);
      }
    });
  });
#pragma unroll
  for (int e = 0; e < E; ++e) { const float2 b3 = lds2<L::B3>(s_w); o0[e] = b3.x; o1[e] = b3.y; }
  static_for<0, H / 2>([&](auto kc) {
    constexpr int k = decltype(kc)::value * 2;
    const float4 w = lds4<L::W3 + 2 * k>(s_w);  // (k: dir, mag), (k+1: dir, mag)
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float ha = fmaxf(h2[e][k], 0.f), hb = fmaxf(h2[e][k + 1], 0.f);
      o0[e] = fmaf(w.x, ha, o0[e]); o1[e] = fmaf(w.y, ha, o1[e]);
      o0[e] = fmaf(w.z, hb, o0[e]); o1[e] = fmaf(w.w, hb, o1[e]);
    }
  });
}

// The parameter's copies in the other ranks' buffers (peer-mapped memory reached by plain stores).
// The pointers are re-read from the descriptor at every store (they sit in L1) rather than held in
// fourteen registers; with n_peer == 0 the cost is one compare.
// n < 0: p[0] is a multicast address that maps every rank's buffer (NVLink switch multicast); one multimem
// store then reaches all of them and the switch does the replication, so the writer's link carries each value
// once instead of once per peer.
struct Peers {
  float* const* p;
  int n;
};
__device__ __forceinline__ Peers load_peers(const pylo_tensor_desc& d) { return Peers{d.p_peer, d.n_peer}; }
__device__ __forceinline__ void peer_store(const Peers& q, int64_t idx, float v) {
  if (q.n < 0) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(q.p[0] + idx), "f"(v) : "memory");
    return;
  }
#pragma unroll 1
  for (int k = 0; k < q.n; ++k) q.p[k][idx] = v;
}
__device__ __forceinline__ void peer_store4(const Peers& q, int64_t idx, float4 v) {
  if (q.n < 0) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(q.p[0] + idx), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
    return;
  }
#pragma unroll 1
  for (int k = 0; k < q.n; ++k) st4(q.p[k] + idx, v);
}

// per-tensor scalars of the output stage, read once per tile
struct Fin {
  float exp_mult, step_mult, wd, lr, lr_eff, param_scale;
  int wd_mode;
};
__device__ __forceinline__ Fin make_fin(const pylo_tensor_desc& d, float param_scale, float lr_eff, int wd_mode) {
  return Fin{d.exp_mult, d.step_mult, d.wd, d.lr, lr_eff, param_scale, wd_mode};
}

template <int FAM>
__device__ __forceinline__ float finish(float p, float o0, float o1, const Fin& c) {
  if (FAM == PYLO_FAM_CELO2) return o0 * __expf(o1 * c.exp_mult);
  if (FAM == PYLO_FAM_ADAFAC) {
    const float upd = o0 * __expf(o1 * c.exp_mult) * c.step_mult;
    float pn = p - c.lr_eff * upd;
    if (c.wd_mode == 1) pn = fmaf(-(c.wd * c.lr), pn, pn);
    else if (c.wd_mode == 2) pn = fmaf(-(c.wd * c.lr), p, pn);
    return pn;
  }
  const float upd = c.param_scale * o0 * __expf(o1 * c.exp_mult) * c.step_mult;
  float pn = p - c.lr_eff * upd;
  if (c.wd > 0.f) pn = pn - c.wd * c.lr_eff * pn;
  return pn;
}

template <int FAM>
__global__ void __launch_bounds__(NT) k_apply(const pylo_tensor_desc* __restrict__ descs,
                                              const pylo_tile* __restrict__ tiles, int n_tiles, int reverse,
                                              const pylo_step_params prm) {
  using F = Fam<FAM>;
  using L = Fold<FAM>;
  constexpr int H = F::H;
  __shared__ __align__(16) float s_w[L::SIZE + 4];
  const int tid = threadIdx.x;
  const uint32_t s_wa = smem_addr(s_w);
  int loaded = -1;
  for (int tt = blockIdx.x; tt < n_tiles; tt += gridDim.x) {
    const int t = reverse ? (n_tiles - 1 - tt) : tt;
    const pylo_tile tl = tiles[t];
    const pylo_tensor_desc& d = descs[tl.tensor];
    if (loaded != tl.tensor) {
      __syncthreads();
      for (int e = tid; e < L::SIZE; e += NT) s_w[e] = d.wfold[e];
      loaded = tl.tensor;
      __syncthreads();
    }
    const int64_t n = d.n, start = tl.start;
    const int cnt = (int)min((int64_t)PYLO_TILE_ELEMS, n - start);
    const float gs = grad_scale_of(d, prm);
    const Fin fin = make_fin(d, s_w[L::SC], s_w[L::SC + 1], prm.wd_mode);
    const Peers peers = load_peers(d);
    const float* gp = d.g + start;
    float* pp = d.p + start;
    float* op = (FAM == PYLO_FAM_CELO2) ? d.out + start : pp;
    const float* m0p = d.m + start;
    const float* m1p = d.m + d.m_stride + start;
    const float* m2p = d.m + 2 * d.m_stride + start;
    const float* vp = d.v + start;

    {
      const Geo geo{(uint32_t)d.X, (uint32_t)d.M, (uint32_t)d.Y, (uint32_t)d.I};
      const bool vec1d = d.mode == PYLO_MODE_VEC1D;
      const int64_t La = vec1d ? n : d.La, Lb = vec1d ? n : d.Lb;
      const float* fac_r = d.r_is_a ? d.fac_a : d.fac_b;
      const float* fac_c = d.r_is_a ? d.fac_b : d.fac_a;
      for (int i = tid; i < cnt; i += NT) {
        const float g = xform_grad(gp[i], gs, prm.clip_val, prm.nan_to_num);
        const float p = pp[i], m0 = m0p[i], m1 = m1p[i], m2 = m2p[i], v = vp[i];
        const float rs = rsqrtf(v + prm.eps_feat);
        float f[1][F::NF];
        if (vec1d) {
          const int64_t e = start + i;
          const float r0 = d.fac_a[e], r1 = d.fac_a[n + e], r2 = d.fac_a[2 * n + e];
          const float* cb = d.fac_b ? d.fac_b : d.fac_a;
          elem_features<FAM>(f[0], g, p, m0, m1, m2, v, rs, safe_rsqrt(r0 + 1e-9f), safe_rsqrt(r1 + 1e-9f), safe_rsqrt(r2 + 1e-9f));
          vec_features<FAM>(f[0], r0, r1, r2, cb[e], cb[n + e], cb[2 * n + e]);
        } else {
          uint64_t a, b;
          geo.split((uint64_t)(d.idx0 + start + i), a, b);
          elem_features<FAM>(f[0], g, p, m0, m1, m2, v, rs, d.f_a[a] * d.f_b[b], d.f_a[La + a] * d.f_b[Lb + b],
                             d.f_a[2 * La + a] * d.f_b[2 * Lb + b]);
          const uint64_t ir = d.r_is_a ? a : b, ic = d.r_is_a ? b : a;
          const int64_t Lr = d.r_is_a ? La : Lb, Lc = d.r_is_a ? Lb : La;
          vec_features<FAM>(f[0], fac_r[ir], fac_r[Lr + ir], fac_r[2 * Lr + ir], fac_c[ic], fac_c[Lc + ic], fac_c[2 * Lc + ic]);
        }
        float h1[1][H], o0[1], o1[1];
#pragma unroll
        for (int j = 0; j < H; ++j) h1[0][j] = s_w[L::B1 + j];
        network<FAM, true, 1>(s_wa, h1, f, o0, o1);
        const float pn = finish<FAM>(p, o0[0], o1[0], fin);
        op[i] = pn;
        if (FAM != PYLO_FAM_CELO2) peer_store(peers, start + i, pn);
      }
    }
  }
}

// ================================================================================================
// Phase C for AdafacLO / ELO on FAST2D tensors: thread-owns-column kernel.
//
// The 39-32-32-2 network costs ~1600 fp32 FMAs per element once the vector-only features and
// the time features are folded away, so this sweep is bound by FMA issue, not by HBM.  Layout:
//   * a CTA takes a tile of RT rows x CW columns; a thread keeps ONE column for all its rows, so
//     the column's tabulated first-layer term (32 floats) and its three column factors stay in
//     registers, and the rows' terms sit in shared memory;
//   * two rows are processed at once so every weight read from shared memory feeds two elements;
//   * all multiply-adds are packed fma.rn.f32x2 (two fp32 FMAs per instruction) over pairs of
//     adjacent hidden units, which halves the issue slots the FMAs need;
//   * the first hidden layer's activations are staged through shared memory so that the second
//     layer can run as a short loop over k instead of 1000+ unrolled instructions;
//   * the next pair's operands are loaded while the current pair is computed.
// ================================================================================================
#define CC_TILE_ROWS 32   // rows per tile

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

#define CC_E 2            // rows a thread processes at once (each weight read feeds CC_E elements)
#define CC_CTAS_PER_SM 2  // 128 registers per thread

__device__ __forceinline__ float ldg_early(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

struct CcSmem {
  float w[Fold<PYLO_FAM_ADAFAC>::SIZE + 12];  // folded network
  float ha[CC_TILE_ROWS][32];                 // first-layer terms of the tile's rows (bias included)
  float fx[CC_TILE_ROWS][4];                  // the rows' three factors
  float hb[16][NT][2];                        // first-layer terms of the tile's columns, hidden-unit pairs
  float h1[32][NT][CC_E];                     // staged first-layer activations of the rows in flight
};

__global__ void __launch_bounds__(NT, CC_CTAS_PER_SM) k_apply_adafac_cols(const pylo_tensor_desc* __restrict__ descs,
                                                              const pylo_atile* __restrict__ ctiles, int n_ctiles,
                                                              const pylo_step_params prm) {
  using F = Fam<PYLO_FAM_ADAFAC>;
  using L = Fold<PYLO_FAM_ADAFAC>;
  constexpr int E = CC_E;
  extern __shared__ __align__(16) unsigned char cc_raw[];
  CcSmem& sm = *reinterpret_cast<CcSmem*>(cc_raw);
  const int tid = threadIdx.x;
  int loaded = -1;
  for (int t = blockIdx.x; t < n_ctiles; t += gridDim.x) {
    const pylo_atile ct = ctiles[t];
    const pylo_tensor_desc& d = descs[ct.tensor];
    const int X = d.X, Y = d.Y;
    const int cw = ct.pad_ & 0xffff;                 // columns per CTA: 32, 64, 128 or 256
    const int n_sub = ct.pad_ >> 16;                 // the work item covers n_sub sub-tiles of CC_TILE_ROWS rows
    const int ng = NT / cw;                          // row groups
    const int rt = CC_TILE_ROWS;                     // rows per sub-tile
    const int rows_per_thread = rt / ng;             // 32, 16, 8 or 4
    const int y0 = ct.cb * cw;
    const int col = tid % cw, rg = tid / cw;
    const int y = y0 + col;
    const bool colok = y < Y;
    const int yc = colok ? y : 0;
    __syncthreads();
    if (loaded != ct.tensor) {
      for (int e = tid; e < L::SIZE; e += NT) sm.w[e] = d.wfold[e];
      loaded = ct.tensor;
    }
    // this column's first-layer term (stored transposed, [32][Y]); each thread keeps its own slot, and it
    // serves every sub-tile of the work item
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
      sm.hb[j][tid][0] = d.h_b[(int64_t)(2 * j) * Y + yc];
      sm.hb[j][tid][1] = d.h_b[(int64_t)(2 * j + 1) * Y + yc];
    }
    const float fb0 = d.f_b[yc], fb1 = d.f_b[Y + yc], fb2 = d.f_b[2 * (int64_t)Y + yc];
    const float gs = grad_scale_of(d, prm);
    const int64_t n = d.n;
    const float* __restrict__ gp = d.g;
    float* __restrict__ pp = d.p;
    const float* __restrict__ mp = d.m;
    const float* __restrict__ vp = d.v;
    const Peers peers = load_peers(d);
    for (int sub = 0; sub < n_sub; ++sub) {
    const int x0 = (ct.strip * n_sub + sub) * rt;
    if (x0 >= X) break;
    __syncthreads();  // the previous sub-tile's rows are no longer read
    for (int e = tid; e < rt * 32; e += NT) {
      const int r = e >> 5, x = x0 + r;
      sm.ha[r][e & 31] = x < X ? d.h_a[(int64_t)x * 32 + (e & 31)] : 0.f;
    }
    for (int e = tid; e < rt * 4; e += NT) {
      const int r = e >> 2, x = x0 + r;
      sm.fx[r][e & 3] = x < X ? d.fx[(int64_t)x * 4 + (e & 3)] : 0.f;
    }
    __syncthreads();
    const Fin fin = make_fin(d, 1.0f, sm.w[L::SC + 1], prm.wd_mode);
    float cg[E], cp[E], cm0[E], cm1[E], cm2[E], cv[E];
    auto load_rows = [&](int q, float* g, float* p, float* m0, float* m1, float* m2, float* v) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int x = x0 + rg + ng * (q + e);
        const bool ok = colok && x < X;
        const int64_t idx = ok ? (int64_t)x * Y + y : 0;
        // issued as volatile loads so that they stay here, a whole row pair ahead of their use
        g[e] = ldg_early(gp + idx); p[e] = ldg_early(pp + idx); m0[e] = ldg_early(mp + idx);
        m1[e] = ldg_early(mp + n + idx); m2[e] = ldg_early(mp + 2 * n + idx); v[e] = ldg_early(vp + idx);
      }
    };
    load_rows(0, cg, cp, cm0, cm1, cm2, cv);
#pragma unroll 1
    for (int q = 0; q < rows_per_thread; q += E) {
      float ng_[E], np_[E], nm0[E], nm1[E], nm2[E], nv[E];
      const bool more = q + E < rows_per_thread;
      if (more) load_rows(q + E, ng_, np_, nm0, nm1, nm2, nv);
      // ---- features of the rows in flight
      float f[E][F::NF];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int r = rg + ng * (q + e);
        const float g = xform_grad(cg[e], gs, prm.clip_val, prm.nan_to_num);
        const float rs = rsqrt_pos(cv[e] + prm.eps_feat);
        const float4 fa = ld4(&sm.fx[r][0]);
        elem_features<PYLO_FAM_ADAFAC>(f[e], g, cp[e], cm0[e], cm1[e], cm2[e], cv[e], rs, fa.x * fb0, fa.y * fb1, fa.z * fb2);
      }
      // ---- first layer in two halves of 16 hidden units
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint64_t h1[E][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t b = *reinterpret_cast<const uint64_t*>(&sm.hb[half * 8 + j][tid][0]);
#pragma unroll
          for (int e = 0; e < E; ++e)
            h1[e][j] = add2(*reinterpret_cast<const uint64_t*>(&sm.ha[rg + ng * (q + e)][half * 16 + 2 * j]), b);
        }
        static_for<0, F::NF>([&](auto kc) {
          constexpr int k = decltype(kc)::value;
          if constexpr (!is_vec_feature<PYLO_FAM_ADAFAC>(k)) {
            uint64_t fk[E];
#pragma unroll
            for (int e = 0; e < E; ++e) fk[e] = pack2(f[e][k], f[e][k]);
            const ulonglong2* wrow = reinterpret_cast<const ulonglong2*>(&sm.w[L::W1 + k * 32 + half * 16]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const ulonglong2 w = wrow[j];
#pragma unroll
              for (int e = 0; e < E; ++e) {
                h1[e][2 * j] = fma2(w.x, fk[e], h1[e][2 * j]);
                h1[e][2 * j + 1] = fma2(w.y, fk[e], h1[e][2 * j + 1]);
              }
            }
          }
        });
        // stage relu(h1), the E rows of one hidden unit side by side, for the second layer's dynamic index
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float lo[E], hi[E];
#pragma unroll
          for (int e = 0; e < E; ++e) { unpack2(h1[e][j], lo[e], hi[e]); lo[e] = fmaxf(lo[e], 0.f); hi[e] = fmaxf(hi[e], 0.f); }
          if constexpr (E == 4) {
            st4(&sm.h1[half * 16 + 2 * j][tid][0], make_float4(lo[0], lo[1], lo[2], lo[3]));
            st4(&sm.h1[half * 16 + 2 * j + 1][tid][0], make_float4(hi[0], hi[1], hi[2], hi[3]));
          } else {
            *reinterpret_cast<float2*>(&sm.h1[half * 16 + 2 * j][tid][0]) = make_float2(lo[0], lo[1]);
            *reinterpret_cast<float2*>(&sm.h1[half * 16 + 2 * j + 1][tid][0]) = make_float2(hi[0], hi[1]);
          }
        }
      }
      // ---- second layer: h2 = b2 + W2^T relu(h1)
      uint64_t h2[E][16];
      {
        const ulonglong2* brow = reinterpret_cast<const ulonglong2*>(&sm.w[L::B2]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const ulonglong2 b = brow[j];
#pragma unroll
          for (int e = 0; e < E; ++e) { h2[e][2 * j] = b.x; h2[e][2 * j + 1] = b.y; }
        }
      }
      {
        // the staged activations of unit k+1 are requested while unit k is multiplied in
        float2 cur = *reinterpret_cast<const float2*>(&sm.h1[0][tid][0]);
#pragma unroll 4
        for (int k = 0; k < 32; ++k) {
          const float2 nxt = *reinterpret_cast<const float2*>(&sm.h1[(k + 1) & 31][tid][0]);
          const uint64_t hk0 = pack2(cur.x, cur.x), hk1 = pack2(cur.y, cur.y);
          const ulonglong2* wrow = reinterpret_cast<const ulonglong2*>(&sm.w[L::W2 + k * 32]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const ulonglong2 w = wrow[j];
            h2[0][2 * j] = fma2(w.x, hk0, h2[0][2 * j]); h2[0][2 * j + 1] = fma2(w.y, hk0, h2[0][2 * j + 1]);
            h2[1][2 * j] = fma2(w.x, hk1, h2[1][2 * j]); h2[1][2 * j + 1] = fma2(w.y, hk1, h2[1][2 * j + 1]);
          }
          cur = nxt;
        }
      }
      // ---- output layer: direction and magnitude as packed dot products over hidden-unit pairs, two
      //      partial accumulators each so that no dependent chain is longer than eight FMAs
      uint64_t od[E][2], om[E][2];
#pragma unroll
      for (int e = 0; e < E; ++e) { od[e][0] = od[e][1] = 0ull; om[e][0] = om[e][1] = 0ull; }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&sm.w[L::W3P + 4 * j]);  // (dir pair, mag pair)
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float a, b;
          unpack2(h2[e][j], a, b);
          const uint64_t r = pack2(fmaxf(a, 0.f), fmaxf(b, 0.f));
          od[e][j & 1] = fma2(w.x, r, od[e][j & 1]);
          om[e][j & 1] = fma2(w.y, r, om[e][j & 1]);
        }
      }
      float o0v[E], o1v[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        float a, b, c, dd;
        unpack2(add2(od[e][0], od[e][1]), a, b);
        unpack2(add2(om[e][0], om[e][1]), c, dd);
        o0v[e] = (a + b) + sm.w[L::B3];
        o1v[e] = (c + dd) + sm.w[L::B3 + 1];
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int x = x0 + rg + ng * (q + e);
        if (colok && x < X) {
          const float pn = finish<PYLO_FAM_ADAFAC>(cp[e], o0v[e], o1v[e], fin);
          pp[(int64_t)x * Y + y] = pn;
          peer_store(peers, (int64_t)x * Y + y, pn);
        }
      }
      if (more) {
#pragma unroll
        for (int e = 0; e < E; ++e) { cg[e] = ng_[e]; cp[e] = np_[e]; cm0[e] = nm0[e]; cm1[e] = nm1[e]; cm2[e] = nm2[e]; cv[e] = nv[e]; }
      }
    }
    }  // sub-tiles
  }
}

#include "pylo_apply_tc.cuh"
#include "pylo_ns_gemm.cuh"

// ================================================================================================
// Phase C for CELO2 / ELO_CELO2 / VeLO on FAST2D tensors: packed kernel.
//
// These networks are small (30-8-8-3, 30-4-4-3), so the sweep should run at HBM speed; what stands
// in the way is the instruction count per element.  This kernel halves it:
//   * all arithmetic is done on PAIRS OF ADJACENT ELEMENTS with packed fp32x2 instructions: a
//     float4 load already is two such pairs, so no register moves are needed to form them;
//   * weights sit in shared memory as (w, w) pairs, one 128-bit read feeds four elements;
//   * a thread keeps four columns for all rows of its tile, so the columns' tabulated first-layer
//     terms and factors stay in registers; the rows' terms arrive as broadcast loads;
//   * the next row's six float4 operands are requested before the current row is computed.
// ================================================================================================
template <int FAM>
struct PkW {  // duplicated-weight layout in shared memory (floats)
  static constexpr int H = Fam<FAM>::H;
  static constexpr int W1 = 0;                   // [30][H] pairs
  static constexpr int W2 = W1 + 30 * H * 2;     // [H][H] pairs, k-major
  static constexpr int B2 = W2 + H * H * 2;      // [H] pairs
  static constexpr int W3 = B2 + H * 2;          // [H][2] pairs
  static constexpr int B3 = W3 + H * 4;          // [2] pairs
  static constexpr int SIZE = B3 + 4;
};

struct PkBase {  // packed per-pair operands the features are made of
  uint64_t g, cg, p, m0, m1, m2, v, rs, k0, k1, k2;
};

template <int K>
__device__ __forceinline__ uint64_t pk_feature(const PkBase& b) {
  if constexpr (K == 0) return b.g;
  else if constexpr (K == 1) return b.cg;
  else if constexpr (K == 2) return b.p;
  else if constexpr (K == 3) return b.m0;
  else if constexpr (K == 4) return b.m1;
  else if constexpr (K == 5) return b.m2;
  else if constexpr (K == 6) return b.v;
  else if constexpr (K == 7) return mul2(b.m0, b.rs);
  else if constexpr (K == 8) return mul2(b.m1, b.rs);
  else if constexpr (K == 9) return mul2(b.m2, b.rs);
  else if constexpr (K == 10) return b.rs;
  else if constexpr (K == 11) return mul2(b.k0, b.g);
  else if constexpr (K == 12) return mul2(b.k1, b.g);
  else if constexpr (K == 13) return mul2(b.k2, b.g);
  else if constexpr (K == 14) return mul2(b.g, b.rs);
  else if constexpr (K == 27) return mul2(b.k0, b.m0);
  else if constexpr (K == 28) return mul2(b.k1, b.m1);
  else return mul2(b.k2, b.m2);
}

#define PK_ROWS 16  // rows per thread in a tile

#ifndef PK_CTAS_VELO
#define PK_CTAS_VELO 2
#endif
template <int FAM>
__global__ void __launch_bounds__(NT, FAM == PYLO_FAM_VELO ? PK_CTAS_VELO : 2) k_apply_packed(const pylo_tensor_desc* __restrict__ descs,
                                                        const pylo_atile* __restrict__ ctiles, int n_ctiles,
                                                        const pylo_step_params prm) {
  using F = Fam<FAM>;
  using L = Fold<FAM>;
  using W = PkW<FAM>;
  constexpr int H = F::H;
  __shared__ __align__(16) float s_w[W::SIZE];
  __shared__ float s_sc[2];
  const int tid = threadIdx.x;
  int loaded = -1;
  for (int t = blockIdx.x; t < n_ctiles; t += gridDim.x) {
    const pylo_atile ct = ctiles[t];
    const pylo_tensor_desc& d = descs[ct.tensor];
    const int X = d.X, Y = d.Y;
    const int tpr = ct.pad_;          // threads per row: 8 .. 256 (a thread owns 4 columns)
    const int ng = NT / tpr;          // row groups
    const int rt = PK_ROWS * ng;      // rows per tile
    const int x0 = ct.strip * rt, y0 = ct.cb * tpr * 4;
    if (loaded != ct.tensor) {
      __syncthreads();
      const float* __restrict__ wf = d.wfold;
      for (int e = tid; e < 30 * H; e += NT) { const float w = wf[L::W1 + e]; s_w[W::W1 + 2 * e] = w; s_w[W::W1 + 2 * e + 1] = w; }
      for (int e = tid; e < H * H; e += NT) { const float w = wf[L::W2 + e]; s_w[W::W2 + 2 * e] = w; s_w[W::W2 + 2 * e + 1] = w; }
      for (int e = tid; e < H; e += NT) { const float w = wf[L::B2 + e]; s_w[W::B2 + 2 * e] = w; s_w[W::B2 + 2 * e + 1] = w; }
      for (int e = tid; e < H * 2; e += NT) { const float w = wf[L::W3 + e]; s_w[W::W3 + 2 * e] = w; s_w[W::W3 + 2 * e + 1] = w; }
      for (int e = tid; e < 2; e += NT) { const float w = wf[L::B3 + e]; s_w[W::B3 + 2 * e] = w; s_w[W::B3 + 2 * e + 1] = w; s_sc[e] = wf[L::SC + e]; }
      loaded = ct.tensor;
      __syncthreads();
    }
    const int y = y0 + 4 * (tid % tpr), rg = tid / tpr;
    const bool colok = y < Y;
    const int yc = colok ? y : 0;
    const Fin fin = make_fin(d, s_sc[0], s_sc[1], prm.wd_mode);
    const float gs = grad_scale_of(d, prm);
    const float eps_feat = prm.eps_feat, clip = prm.clip_val;
    const int64_t n = d.n;
    // the four columns' first-layer terms and factors: pairs (col, col+1) and (col+2, col+3)
    uint64_t hb[2][H], fb[2][3];
#pragma unroll
    for (int j = 0; j < H; ++j) {
      const float4 q = ld4(d.h_b + (int64_t)j * Y + yc);
      hb[0][j] = pack2(q.x, q.y);
      hb[1][j] = pack2(q.z, q.w);
    }
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const float4 q = ld4(d.f_b + (int64_t)k * Y + yc);
      fb[0][k] = pack2(q.x, q.y);
      fb[1][k] = pack2(q.z, q.w);
    }
    const float* __restrict__ gp = d.g;
    float* __restrict__ pp = d.p;
    float* __restrict__ op = (FAM == PYLO_FAM_CELO2) ? d.out : d.p;
    const float* __restrict__ mp = d.m;
    const float* __restrict__ vp = d.v;
    const float* __restrict__ hap = d.h_a;
    const float* __restrict__ fxp = d.fx;
    const Peers peers = load_peers(d);

    float4 cg, cp, cm0, cm1, cm2, cv;
    auto load_row = [&](int q, float4& g, float4& p, float4& m0, float4& m1, float4& m2, float4& v) {
      const int x = x0 + rg + ng * q;
      const int64_t idx = (colok && x < X) ? (int64_t)x * Y + y : 0;
      g = ldg4(gp + idx); p = ld4(pp + idx); m0 = ld4(mp + idx); m1 = ld4(mp + n + idx); m2 = ld4(mp + 2 * n + idx); v = ld4(vp + idx);
    };
    load_row(0, cg, cp, cm0, cm1, cm2, cv);
#pragma unroll 1
    for (int q = 0; q < PK_ROWS; ++q) {
      float4 ng_, np_, nm0, nm1, nm2, nv;
      if (q + 1 < PK_ROWS) load_row(q + 1, ng_, np_, nm0, nm1, nm2, nv);
      const int x = x0 + rg + ng * q;
      const int xc = x < X ? x : 0;
      const float4 fa = ld4(fxp + 4 * (int64_t)xc);
      PkBase b[2];
      {
        float ge[4] = {cg.x, cg.y, cg.z, cg.w};
        float rs[4] = {rsqrt_pos(cv.x + eps_feat), rsqrt_pos(cv.y + eps_feat), rsqrt_pos(cv.z + eps_feat), rsqrt_pos(cv.w + eps_feat)};
        float cl[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { ge[u] = xform_grad(ge[u], gs, clip, prm.nan_to_num); cl[u] = fminf(fmaxf(ge[u], -0.1f), 0.1f); }
        const uint64_t a0 = pack2(fa.x, fa.x), a1 = pack2(fa.y, fa.y), a2 = pack2(fa.z, fa.z);
        b[0] = PkBase{pack2(ge[0], ge[1]), pack2(cl[0], cl[1]), pack2(cp.x, cp.y), pack2(cm0.x, cm0.y), pack2(cm1.x, cm1.y),
                      pack2(cm2.x, cm2.y), pack2(cv.x, cv.y), pack2(rs[0], rs[1]), mul2(a0, fb[0][0]), mul2(a1, fb[0][1]), mul2(a2, fb[0][2])};
        b[1] = PkBase{pack2(ge[2], ge[3]), pack2(cl[2], cl[3]), pack2(cp.z, cp.w), pack2(cm0.z, cm0.w), pack2(cm1.z, cm1.w),
                      pack2(cm2.z, cm2.w), pack2(cv.z, cv.w), pack2(rs[2], rs[3]), mul2(a0, fb[1][0]), mul2(a1, fb[1][1]), mul2(a2, fb[1][2])};
      }
      // first layer: h1 = (row term + column term) + sum_k W1[k] f_k
      uint64_t h1[2][H];
#pragma unroll
      for (int j = 0; j < H; j += 2) {
        const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(hap + ((int64_t)xc * H + j) * 2);
        h1[0][j] = add2(hb[0][j], a.x); h1[0][j + 1] = add2(hb[0][j + 1], a.y);
        h1[1][j] = add2(hb[1][j], a.x); h1[1][j + 1] = add2(hb[1][j + 1], a.y);
      }
      static_for<0, F::NF>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        if constexpr (!is_vec_feature<FAM>(k)) {
          const uint64_t f0 = pk_feature<k>(b[0]), f1 = pk_feature<k>(b[1]);
#pragma unroll
          for (int j = 0; j < H; j += 2) {
            const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&s_w[W::W1 + (k * H + j) * 2]);
            h1[0][j] = fma2(w.x, f0, h1[0][j]); h1[0][j + 1] = fma2(w.y, f0, h1[0][j + 1]);
            h1[1][j] = fma2(w.x, f1, h1[1][j]); h1[1][j + 1] = fma2(w.y, f1, h1[1][j + 1]);
          }
        }
      });
      // second layer
      uint64_t h2[2][H];
#pragma unroll
      for (int j = 0; j < H; j += 2) {
        const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(&s_w[W::B2 + j * 2]);
        h2[0][j] = bb.x; h2[0][j + 1] = bb.y; h2[1][j] = bb.x; h2[1][j + 1] = bb.y;
      }
      static_for<0, H>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        uint64_t r[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float lo, hi;
          unpack2(h1[e][k], lo, hi);
          r[e] = pack2(fmaxf(lo, 0.f), fmaxf(hi, 0.f));
        }
#pragma unroll
        for (int j = 0; j < H; j += 2) {
          const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&s_w[W::W2 + (k * H + j) * 2]);
          h2[0][j] = fma2(w.x, r[0], h2[0][j]); h2[0][j + 1] = fma2(w.y, r[0], h2[0][j + 1]);
          h2[1][j] = fma2(w.x, r[1], h2[1][j]); h2[1][j + 1] = fma2(w.y, r[1], h2[1][j + 1]);
        }
      });
      // output layer: direction and magnitude
      const ulonglong2 b3 = *reinterpret_cast<const ulonglong2*>(&s_w[W::B3]);
      uint64_t o0[2] = {b3.x, b3.x}, o1[2] = {b3.y, b3.y};
      static_for<0, H>([&](auto kc) {
        constexpr int k = decltype(kc)::value;
        const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&s_w[W::W3 + k * 4]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float lo, hi;
          unpack2(h2[e][k], lo, hi);
          const uint64_t r = pack2(fmaxf(lo, 0.f), fmaxf(hi, 0.f));
          o0[e] = fma2(w.x, r, o0[e]);
          o1[e] = fma2(w.y, r, o1[e]);
        }
      });
      if (colok && x < X) {
        float d0, d1, d2, d3, m0, m1, m2, m3;
        unpack2(o0[0], d0, d1); unpack2(o0[1], d2, d3);
        unpack2(o1[0], m0, m1); unpack2(o1[1], m2, m3);
        const float4 res = make_float4(finish<FAM>(cp.x, d0, m0, fin), finish<FAM>(cp.y, d1, m1, fin),
                                       finish<FAM>(cp.z, d2, m2, fin), finish<FAM>(cp.w, d3, m3, fin));
        st4(op + (int64_t)x * Y + y, res);
        if (FAM != PYLO_FAM_CELO2) peer_store4(peers, (int64_t)x * Y + y, res);
      }
      if (q + 1 < PK_ROWS) { cg = ng_; cp = np_; cm0 = nm0; cm1 = nm1; cm2 = nm2; cv = nv; }
    }
  }
}

// ================================================================================================
// CELO2 tail: second-moment normaliser over a matrix, then the parameter update
// ================================================================================================
__global__ void __launch_bounds__(NT) k_post_sums(const pylo_post_item* __restrict__ items,
                                                  const pylo_tile* __restrict__ tiles, int n_tiles) {
  __shared__ float s_red[40];
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const pylo_tile tl = tiles[t];
    const pylo_post_item& it = items[tl.tensor];
    const float* s = it.step + tl.start;
    const int cnt = (int)min((int64_t)PYLO_TILE_ELEMS, it.n - tl.start);
    float acc = 0.f;
    if (((((uintptr_t)s) & 15) == 0)) {
      const int c4 = cnt & ~3;
      for (int i = threadIdx.x * 4; i < c4; i += NT * 4) {
        const float4 q = ld4(s + i);
        acc += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
      }
      for (int i = c4 + threadIdx.x; i < cnt; i += NT) acc += s[i] * s[i];
    } else {
      for (int i = threadIdx.x; i < cnt; i += NT) acc += s[i] * s[i];
    }
    const float tot = block_sum(acc, s_red);
    if (threadIdx.x == 0) it.part[t - it.tile0] = tot;
  }
}

__global__ void __launch_bounds__(NT) k_post_apply(const pylo_post_item* __restrict__ items,
                                                   const pylo_tile* __restrict__ tiles, int n_tiles) {
  __shared__ float s_scale;
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const pylo_tile tl = tiles[t];
    const pylo_post_item& it = items[tl.tensor];
    __syncthreads();
    if (threadIdx.x < 32) {  // every tile re-reduces the item's partials in the same fixed order
      double acc = 0.0;
      for (int q = threadIdx.x; q < it.n_tiles; q += 32) acc += (double)it.part[q];
      acc = warp_sum_d(acc);
      if (threadIdx.x == 0) s_scale = rsqrtf(1e-9f + (float)acc / (float)it.n) * it.rmsmult;
    }
    __syncthreads();
    const float sc = s_scale, lr = it.lr, wd = it.wd;
    const float* s = it.step + tl.start;
    float* p = it.p + tl.start;
    const int cnt = (int)min((int64_t)PYLO_TILE_ELEMS, it.n - tl.start);
    const bool al = (((((uintptr_t)s) | ((uintptr_t)p)) & 15) == 0);
    const int c4 = al ? (cnt & ~3) : 0;
    for (int i = threadIdx.x * 4; i < c4; i += NT * 4) {
      const float4 q = ld4(s + i);
      float4 w = ld4(p + i);
      w.x = fmaf(-lr, fmaf(q.x, sc, wd * w.x), w.x);
      w.y = fmaf(-lr, fmaf(q.y, sc, wd * w.y), w.y);
      w.z = fmaf(-lr, fmaf(q.z, sc, wd * w.z), w.z);
      w.w = fmaf(-lr, fmaf(q.w, sc, wd * w.w), w.w);
      st4(p + i, w);
    }
    for (int i = c4 + threadIdx.x; i < cnt; i += NT) p[i] = fmaf(-lr, fmaf(s[i], sc, wd * p[i]), p[i]);
  }
}

// ================================================================================================
// AdamW branch
// ================================================================================================
__global__ void __launch_bounds__(NT) k_adamw(const pylo_adam_item* __restrict__ items,
                                              const pylo_tile* __restrict__ tiles, int n_tiles, int independent,
                                              float beta1, float omb1, float beta2, float omb2, float eps,
                                              const pylo_step_params prm) {
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const pylo_tile tl = tiles[t];
    const pylo_adam_item& it = items[tl.tensor];
    const int64_t n = it.n;
    const int cnt = (int)min((int64_t)PYLO_TILE_ELEMS, n - tl.start);
    float gs = 1.0f;
    if (it.clip_norm > 0.f && prm.gnorm_sq) {
      const float denom = fmaxf(sqrtf(*prm.gnorm_sq), it.clip_norm);
      gs = denom > 0.f ? it.clip_norm / denom : 1.0f;
    }
    const float* gp = it.g + tl.start;
    float* pp = it.p + tl.start;
    float* vp = it.v + tl.start;
    float* mp = it.m + tl.start;
    for (int i = threadIdx.x; i < cnt; i += NT) {
      const float g = xform_grad(gp[i], gs, prm.clip_val, prm.nan_to_num);
      const float p = pp[i];
      float m, v;
      if (independent) {  // exp_avg.mul_(b1).add_(g, alpha=1-b1); exp_avg_sq.mul_(b2).addcmul_(g, g, value=1-b2)
        m = fmaf(g, omb1, mp[i] * beta1);
        v = fmaf(g * g, omb2, vp[i] * beta2);
        mp[i] = m;
      } else {  // shared accumulators: all three momenta advance, the step uses decay 0
        m = lerp_torch(mp[i], g, prm.w_m[0]);
        mp[i] = m;
        mp[n + i] = lerp_torch(mp[n + i], g, prm.w_m[1]);
        mp[2 * n + i] = lerp_torch(mp[2 * n + i], g, prm.w_m[2]);
        v = lerp_torch(vp[i], g * g, prm.w_v);
      }
      vp[i] = v;
      const float upd = (m / it.bc1) / (sqrtf(v / it.bc2) + eps);
      pp[i] = fmaf(-it.lr, fmaf(it.wd, p, upd), p);
    }
  }
}

// ================================================================================================
// VeLO front end
// ================================================================================================
__device__ __forceinline__ float clip_log_abs10(float v) {
  return fminf(fmaxf(logf(1e-8f + fabsf(v * 10.0f)), -5.f), 5.f) * 0.5f;
}

// one thread per tensor: the 30 LSTM inputs from the statistics gathered in phase B (velo_cuda.py:213-252)
__global__ void k_velo_tensor_features(const pylo_tensor_desc* __restrict__ descs, int n_local,
                                       const int32_t* __restrict__ layer_of, int T,
                                       const float* __restrict__ rank_onehot, const float* __restrict__ fraction9,
                                       const float* __restrict__ loss9, float* __restrict__ x_in) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_local) return;
  const int layer = layer_of ? layer_of[t] : t;  // position of this tensor among all T tensors of the model
  const pylo_tensor_desc& d = descs[t];
  const double n = (double)d.n;
  auto stat = [&](int j) { return (double)d.sums[30 + j] + (double)d.sums[SUMS_LO + j]; };
  const float mean_p2 = (float)((double)d.sums[2] / n);
  const double norm = (double)rsqrtf(fmaxf(mean_p2, 1e-9f));
  float* o = x_in + (int64_t)(T - 1 - layer) * 30;  // rows are flipped (velo_cuda.py:422)
#pragma unroll
  for (int j = 0; j < 9; ++j) { o[j] = fraction9[j]; o[9 + j] = loss9[j]; }
  const double mean_v = stat(6) / n, e_v2 = stat(7) / n;
  o[18] = clip_log_abs10((float)(norm * mean_v));
#pragma unroll
  for (int j = 0; j < 5; ++j) o[19 + j] = rank_onehot[t * 5 + j];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const double mu = stat(k) / n, e_m2 = stat(3 + k) / n;
    const double var_m = fmax(e_m2 - mu * mu, 0.0);
    const double var_v = fmax(e_v2 - 2.0 * mu * mean_v + mu * mu, 0.0);  // mean((rms - mean_m)^2), velo_cuda.py:243
    o[24 + k] = clip_log_abs10((float)(norm * norm * var_m));
    o[27 + k] = clip_log_abs10((float)(norm * norm * var_v));
  }
}

// BufferLossAccumulators.update followed by .features (velo_cuda.py:183-211); one warp
__global__ void k_velo_loss(float* means, int32_t* iteration, float* running_min, const float* __restrict__ decays,
                            const float* __restrict__ loss_in, float* __restrict__ loss9) {
  __shared__ float s_cor[10];
  const int j = threadIdx.x;
  const int it = *iteration;
  float cor = -CUDART_INF_F;
  if (j < 10) cor = means[j] / (1.0f - powf(decays[j], (float)(it + 1)));
  float mx = cor;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float approx_max = it == 0 ? loss_in[0] : mx;
  const float loss = fminf(fabsf(approx_max) * 2.0f, loss_in[0]);
  if (j < 10) {
    const float dj = decays[j];
    const float mnew = means[j] * dj + loss * (1.0f - dj);
    const float c2 = mnew / (1.0f - powf(dj, (float)(it + 1)));
    const float rmin = fminf(running_min[j], c2);
    means[j] = mnew;
    running_min[j] = rmin;
    s_cor[j] = mnew / (1.0f - powf(dj, (float)(it + 1)));  // features() uses iteration after the increment
  }
  __syncwarp();
  if (j < 9) {
    const float rmin = running_min[j];
    const float den = fmaxf(1e-8f, s_cor[j + 1] - rmin);
    float f = fminf(fmaxf((s_cor[j] - rmin) / den - 1.0f, -1.f), 1.f);
    loss9[j] = (it + 1 <= 2) ? f * 0.f : f;
  }
  __syncwarp();
  if (j == 0) *iteration = it + 1;
}

// x' = final_mix(x) + max_t relu(mix2(x)) ; two kernels: pooled (one thread per hidden unit), then xmix
__global__ void k_velo_pool(const pylo_velo_rnn r) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= r.H) return;
  float w[30];
#pragma unroll
  for (int k = 0; k < 30; ++k) w[k] = r.mix2_w[h * 30 + k];
  const float b = r.mix2_b[h];
  float best = -CUDART_INF_F;
  for (int t = 0; t < r.T; ++t) {
    float acc = b;
#pragma unroll
    for (int k = 0; k < 30; ++k) acc = fmaf(w[k], r.x_in[t * 30 + k], acc);
    best = fmaxf(best, fmaxf(acc, 0.f));
  }
  r.pooled[h] = best;
}

__global__ void k_velo_xmix(const pylo_velo_rnn r) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (int64_t)r.T * r.H) return;
  const int t = (int)(e / r.H), h = (int)(e % r.H);
  float acc = r.fmix_b[h];
#pragma unroll
  for (int k = 0; k < 30; ++k) acc = fmaf(r.fmix_w[h * 30 + k], r.x_in[t * 30 + k], acc);
  r.xmix[e] = acc + r.pooled[h];
}

// gates[t][q] = lstm_b[q] + sum_k lstm_w[q][k] * cat(x', h)[t][k]: a [T x 2H] x [2H x 4H] product.
// Shared-memory tiled, 64 x 64 outputs per CTA, 16 deep, 4 x 4 outputs per thread; fp32 throughout
// (the whole product is ~1 GFLOP, far too small to be worth a tensor-core path).
#define GT 64
#define GK 16
__global__ void __launch_bounds__(NT) k_velo_gates(const pylo_velo_rnn r) {
  __shared__ float s_a[GK][GT + 4];
  __shared__ float s_w[GK][GT + 4];
  const int H = r.H, Q = 4 * H, K = 2 * H, T = r.T;
  const int t0 = blockIdx.y * GT, q0 = blockIdx.x * GT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GK) {
    // each thread loads 4 elements of each operand tile: rows (threadIdx.x / 16 + 16 * u), column threadIdx.x % 16
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int row = ty + 16 * u, kk = k0 + tx;
      const int t = t0 + row, q = q0 + row;
      float av = 0.f, wv = 0.f;
      if (t < T && kk < K) av = kk < H ? r.xmix[(int64_t)t * H + kk] : r.h[(int64_t)t * H + (kk - H)];
      if (q < Q && kk < K) wv = r.lstm_w[(int64_t)q * K + kk];
      s_a[tx][row] = av;
      s_w[tx][row] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      const float4 a = ld4(&s_a[kk][ty * 4]);
      const float4 w = ld4(&s_w[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = q0 + tx * 4 + j;
      if (q < Q) r.gates[(int64_t)t * Q + q] = acc[i][j] + r.lstm_b[q];
    }
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// cell update; gate order i, g, f, o with f + 1 (VeLO_RNN.py:57-65)
__global__ void k_velo_cell(const pylo_velo_rnn r) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (int64_t)r.T * r.H) return;
  const int t = (int)(e / r.H), h = (int)(e % r.H), H = r.H;
  const float* g4 = r.gates + (int64_t)t * 4 * H;
  const float i = sigmoidf_(g4[h]), g = tanhf(g4[H + h]), f = sigmoidf_(g4[2 * H + h] + 1.0f), o = sigmoidf_(g4[3 * H + h]);
  const float c = f * r.c[e] + i * g;
  r.c[e] = c;
  r.h[e] = o * tanhf(c);
}

// controls[t][b] and lr_mult[t]; one warp per output
__global__ void __launch_bounds__(NT) k_velo_heads(const pylo_velo_rnn r) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t)blockIdx.x * NWARP + (threadIdx.x >> 5);
  const int H = r.H, B1 = r.B + 1;
  if (wid >= (int64_t)r.T * B1) return;
  const int t = (int)(wid / B1), b = (int)(wid % B1);
  const float* wrow = b < r.B ? r.ctrl_w + (int64_t)b * H : r.step_w;
  float acc = 0.f;
  for (int k = lane; k < H; k += 32) acc = fmaf(wrow[k], r.h[(int64_t)t * H + k], acc);
  acc = warp_sum(acc);
  if (lane == 0) {
    if (b < r.B) r.controls[(int64_t)t * r.B + b] = acc + r.ctrl_b[b];
    else r.lr_mult[r.T - 1 - t] = acc + r.step_b[0];  // row t of the flipped input belongs to tensor T-1-t
  }
}

// weights[tensor][e] = mean_b(control[b] * bank[b][e]) * 100 (VeLO_MLP.py:92-126); block per tensor
__global__ void __launch_bounds__(160) k_velo_mix(const pylo_velo_rnn r) {
  extern __shared__ float s_ctrl[];
  const int tensor = blockIdx.x;
  const int row = r.T - 1 - tensor;
  for (int b = threadIdx.x; b < r.B; b += blockDim.x) s_ctrl[b] = r.controls[(int64_t)row * r.B + b];
  __syncthreads();
  const int e = threadIdx.x;
  if (e < 159) {
    float acc = 0.f;
    for (int b = 0; b < r.B; ++b) acc = fmaf(s_ctrl[b], r.bank[(int64_t)b * 159 + e], acc);
    r.weights[(int64_t)tensor * 160 + e] = acc / (float)r.B * 100.0f;
  }
}

// ================================================================================================
// C ABI
// ================================================================================================
// Opt-in limits and caches are kept per device: the library may be used on every GPU of a box from one process.
#define PYLO_MAX_DEVICES 64
static int g_sm_count[PYLO_MAX_DEVICES] = {0};
static int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PYLO_MAX_DEVICES) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}
static int grid_for(int n_items, int ctas_per_sm) {
  const int cap = sm_count() * ctas_per_sm;
  return n_items < cap ? n_items : cap;
}
static int launch_status() { return (int)cudaGetLastError(); }

// Opt a kernel in to more than 48 KB of dynamic shared memory, once per device (the attribute belongs to the
// device's copy of the function); flags[] is the caller's per-kernel record.
template <class K>
static int allow_dynamic_smem(K kernel, int bytes, bool (&flags)[PYLO_MAX_DEVICES]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < PYLO_MAX_DEVICES && flags[dev]) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < PYLO_MAX_DEVICES) flags[dev] = true;
  return 0;
}

#define CHECK_ARG(cond) \
  do {                  \
    if (!(cond)) return -1; \
  } while (0)

extern "C" {

int pylo_b200_abi_version(void) { return PYLO_B200_ABI_VERSION; }
int pylo_b200_sizeof_desc(void) { return (int)sizeof(pylo_tensor_desc); }
int pylo_b200_sizeof_params(void) { return (int)sizeof(pylo_step_params); }

int pylo_b200_workspace_layout(int family, int mode, int64_t n, int64_t La, int64_t Lb, int32_t X, int32_t Y,
                               pylo_ws_layout* out) {
  CHECK_ARG(out && n > 0);
  CHECK_ARG(family == PYLO_FAM_ADAFAC || family == PYLO_FAM_CELO2 || family == PYLO_FAM_VELO);
  CHECK_ARG(mode == PYLO_MODE_FAST2D || mode == PYLO_MODE_GENERIC || mode == PYLO_MODE_VEC1D);
  const int64_t H = family == PYLO_FAM_ADAFAC ? 32 : (family == PYLO_FAM_CELO2 ? 8 : 4);
  pylo_ws_layout w = {};
  if (mode != PYLO_MODE_VEC1D) {
    CHECK_ARG(La > 0 && Lb > 0);
    w.f_a = 3 * La; w.f_b = 3 * Lb; w.sum_a = La; w.sum_b = Lb;
  }
  if (mode == PYLO_MODE_FAST2D) {
    CHECK_ARG(X > 0 && Y > 0 && Y % 4 == 0 && La == X && Lb == Y);
    int rb = (((X + 127) / 128 + 7) / 8) * 8;  // rows per strip: about X / 128, a multiple of 8, within [32, 128]
    rb = rb < 32 ? 32 : (rb > 128 ? 128 : rb);
    w.rb = rb;
    w.n_strips = (X + rb - 1) / rb;
    w.n_cb = (Y + PYLO_A_COLS - 1) / PYLO_A_COLS;
    w.fx = 4 * La;
    w.part_a = (int64_t)X * w.n_cb;
    w.part_b = (int64_t)w.n_strips * Y;
    w.h_a = La * H * 2;
    w.h_b = Lb * H;
  }
  w.closed = PYLO_STAT_STRIDE;
  w.n_tiles = (int32_t)((n + PYLO_TILE_ELEMS - 1) / PYLO_TILE_ELEMS);
  w.sums = SUMS_STRIDE;
  w.wfold = PYLO_WFOLD_STRIDE;
  w.tile_part = (int64_t)w.n_tiles * PYLO_STAT_STRIDE;
  *out = w;
  return 0;
}

int64_t pylo_b200_workspace_bytes(const pylo_ws_layout* w, int tensor_part, int unit_part) {
  if (!w) return -1;
  auto pad = [](int64_t floats) { return (floats + 63) / 64 * 64 * 4; };
  int64_t bytes = 0;
  if (tensor_part)
    bytes += pad(w->f_a) + pad(w->f_b) + pad(w->sum_a) + pad(w->sum_b) + pad(w->fx) + pad(w->part_a) + pad(w->part_b) +
             pad(w->h_a) + pad(w->h_b) + pad(w->closed);
  if (unit_part) bytes += pad(w->sums) + pad(w->wfold) + pad(w->tile_part);
  return bytes;
}

int pylo_b200_grad_sumsq(const pylo_gvec* descs, const pylo_tile* tiles, int n_tiles, float* scratch,
                         float* out, void* stream) {
  CHECK_ARG(descs && tiles && scratch && out && n_tiles >= 0);
  cudaStream_t s = (cudaStream_t)stream;
  if (n_tiles > 0) k_grad_sumsq<<<grid_for(n_tiles, 8), NT, 0, s>>>(descs, tiles, n_tiles, scratch);
  k_sum_final<<<1, 1024, 0, s>>>(scratch, n_tiles, out);
  return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of pylo_b200_grad_sumsq.
//
// Some hosts of this library cannot hand it scratch memory: a language binding that links only this
// .so and has no device allocator of its own, or a step loop whose rules forbid cudaMalloc because it
// synchronises the device.  For them the per-tile partial sums live in the fixed array below instead
// of a caller buffer.  The array is part of the loaded module, so every GPU that loads the library
// carries its 256 KiB until the process exits.
//
// In host code the name `g_static_sumsq_scratch` is only a handle for the symbol, not a pointer the
// device can follow, so the device address is looked up with cudaGetSymbolAddress, once per device,
// with that device current, and that address is what the kernels receive.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_static_sumsq_scratch[PYLO_STATIC_SCRATCH_TILES];

static float* g_static_scratch_addr[PYLO_MAX_DEVICES] = {nullptr};
static std::mutex g_static_scratch_mutex;

static int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= PYLO_MAX_DEVICES) return -3;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_sumsq_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return -3;
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return 0;
}

int pylo_b200_grad_sumsq_static(const pylo_gvec* items, const pylo_tile* tiles, int n_tiles, float* out,
                                void* stream) {
  CHECK_ARG(items && tiles && out && n_tiles >= 0);
  if (n_tiles > PYLO_STATIC_SCRATCH_TILES) return PYLO_ERR_STATIC_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // every slot that the final sum reads is written by the partial kernel of this same call, so
  // nothing left over from an earlier call needs clearing
  if (n_tiles > 0) k_grad_sumsq<<<grid_for(n_tiles, 8), NT, 0, s>>>(items, tiles, n_tiles, scratch);
  k_sum_final<<<1, 1024, 0, s>>>(scratch, n_tiles, out);
  return launch_status();
}

int pylo_b200_rowcol_sums(const pylo_tensor_desc* descs, const pylo_atile* atiles, int n_atiles,
                          const pylo_atile* rtiles, int n_rtiles, const int32_t* generic_ids, int n_generic,
                          const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && prm && n_atiles >= 0 && n_rtiles >= 0 && n_generic >= 0);
  cudaStream_t s = (cudaStream_t)stream;
  if (n_atiles > 0) {
    CHECK_ARG(atiles && rtiles && n_rtiles > 0);
    k_rowcol_fast<<<grid_for(n_atiles, 4), NT, 0, s>>>(descs, atiles, n_atiles, *prm);
    k_colpart_reduce<<<grid_for(n_rtiles, 8), NT, 0, s>>>(descs, rtiles, n_rtiles);
  }
  if (n_generic > 0) {
    CHECK_ARG(generic_ids);
    k_rowcol_generic<<<n_generic * 16, NT, 0, s>>>(descs, generic_ids, 16, *prm);
  }
  return launch_status();
}

int pylo_b200_factor_update(const pylo_tensor_desc* descs, int n_tensors, const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && prm && n_tensors >= 0);
  if (n_tensors == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  switch (prm->family) {
    case PYLO_FAM_ADAFAC: k_factor_update<PYLO_FAM_ADAFAC><<<n_tensors, A2_NT, 0, s>>>(descs, *prm); break;
    case PYLO_FAM_CELO2: k_factor_update<PYLO_FAM_CELO2><<<n_tensors, A2_NT, 0, s>>>(descs, *prm); break;
    case PYLO_FAM_VELO: k_factor_update<PYLO_FAM_VELO><<<n_tensors, A2_NT, 0, s>>>(descs, *prm); break;
    default: return -2;
  }
  return launch_status();
}

int pylo_b200_state_moments(const pylo_tensor_desc* descs, const pylo_tile* tiles, int n_tiles, int reverse,
                            const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && tiles && prm && n_tiles >= 0);
  if (n_tiles == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = grid_for(n_tiles, 4);
  switch (prm->family) {
    case PYLO_FAM_ADAFAC: k_state_moments<PYLO_FAM_ADAFAC><<<grid, NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    case PYLO_FAM_CELO2: k_state_moments<PYLO_FAM_CELO2><<<grid, NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    case PYLO_FAM_VELO: k_state_moments<PYLO_FAM_VELO><<<grid, NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    default: return -2;
  }
  return launch_status();
}

int pylo_b200_finalize_moments(const pylo_tensor_desc* descs, int n_tensors, void* stream) {
  CHECK_ARG(descs && n_tensors >= 0);
  if (n_tensors == 0) return 0;
  k_finalize_moments<<<n_tensors, NT, 0, (cudaStream_t)stream>>>(descs);
  return launch_status();
}

int pylo_b200_prep_apply(const pylo_tensor_desc* descs, int n_tensors, const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && prm && n_tensors >= 0);
  if (n_tensors == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  // the table loops stride over grid.y slices; with few tensors in a launch the slices are what fills the GPU
  const dim3 grid(n_tensors, n_tensors >= 64 ? 8 : 48);
  switch (prm->family) {
    case PYLO_FAM_ADAFAC: k_prep_apply<PYLO_FAM_ADAFAC><<<grid, NT, 0, s>>>(descs, *prm); break;
    case PYLO_FAM_CELO2: k_prep_apply<PYLO_FAM_CELO2><<<grid, NT, 0, s>>>(descs, *prm); break;
    case PYLO_FAM_VELO: k_prep_apply<PYLO_FAM_VELO><<<grid, NT, 0, s>>>(descs, *prm); break;
    default: return -2;
  }
  return launch_status();
}

int pylo_b200_apply(const pylo_tensor_desc* descs, const pylo_tile* tiles, int n_tiles, int reverse,
                    const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && tiles && prm && n_tiles >= 0);
  if (n_tiles == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  switch (prm->family) {
    case PYLO_FAM_ADAFAC: k_apply<PYLO_FAM_ADAFAC><<<grid_for(n_tiles, 2), NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    case PYLO_FAM_CELO2: k_apply<PYLO_FAM_CELO2><<<grid_for(n_tiles, 4), NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    case PYLO_FAM_VELO: k_apply<PYLO_FAM_VELO><<<grid_for(n_tiles, 4), NT, 0, s>>>(descs, tiles, n_tiles, reverse, *prm); break;
    default: return -2;
  }
  return launch_status();
}

int pylo_b200_apply_adafac_cols(const pylo_tensor_desc* descs, const pylo_atile* ctiles, int n_ctiles,
                                const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && ctiles && prm && n_ctiles >= 0 && prm->family == PYLO_FAM_ADAFAC);
  if (n_ctiles == 0) return 0;
  static bool configured[PYLO_MAX_DEVICES] = {};
  if (int rc = allow_dynamic_smem(k_apply_adafac_cols, (int)sizeof(CcSmem), configured)) return rc;
  k_apply_adafac_cols<<<grid_for(n_ctiles, CC_CTAS_PER_SM), NT, sizeof(CcSmem), (cudaStream_t)stream>>>(descs, ctiles, n_ctiles, *prm);
  return launch_status();
}

int pylo_b200_apply_adafac_tc(const pylo_tensor_desc* descs, const pylo_atile* ttiles, int n_ttiles,
                              const pylo_step_params* prm, int* status, void* stream) {
  CHECK_ARG(descs && ttiles && prm && n_ttiles >= 0 && prm->family == PYLO_FAM_ADAFAC);
  if (n_ttiles == 0) return 0;
  // more than half an SM's shared memory is requested: one CTA per SM, which then owns all of the SM's tensor memory
  constexpr int smem = sizeof(TcSmem) > 120 * 1024 ? (int)sizeof(TcSmem) : 120 * 1024;
  static bool configured[PYLO_MAX_DEVICES] = {};
  if (int rc = allow_dynamic_smem(k_apply_adafac_tc, smem, configured)) return rc;
  k_apply_adafac_tc<<<grid_for(n_ttiles, 1), TC_NT, smem, (cudaStream_t)stream>>>(descs, ttiles, n_ttiles, *prm, status);
  return launch_status();
}

int pylo_b200_gemm_tn_3xtf32(const pylo_gemm_desc* g, int* status, void* stream) {
  CHECK_ARG(g && g->A && g->B && g->C);
  CHECK_ARG(g->M > 0 && g->N > 0 && g->K > 0 && g->batch > 0);
  // rows are moved in 16-byte pieces
  CHECK_ARG(g->K % 4 == 0 && g->N % 4 == 0 && g->lda % 4 == 0 && g->ldb % 4 == 0 && g->ldc % 4 == 0);
  CHECK_ARG(g->lda >= g->K && g->ldb >= g->K && g->ldc >= g->N);
  CHECK_ARG(((uintptr_t)g->A | (uintptr_t)g->B | (uintptr_t)g->C | (uintptr_t)g->D) % 16 == 0);
  CHECK_ARG(g->strideA % 4 == 0 && g->strideB % 4 == 0 && g->strideC % 4 == 0);
  if (g->D) CHECK_ARG(g->ldd % 4 == 0 && g->ldd >= g->N && g->strideD % 4 == 0 && g->D != g->C);
  static_assert(sizeof(pylo_gemm_desc) == sizeof(pylo_gemm_args), "pylo_gemm_desc and the kernel's argument block differ");
  pylo_gemm_args a;
  memcpy(&a, g, sizeof(a));
  if (g->symmetric) CHECK_ARG(g->M == g->N);
  const long long tiles = (long long)ns_tiles_per_matrix((g->M + NS_BM - 1) / NS_BM, (g->N + NS_BN - 1) / NS_BN, g->symmetric) * g->batch;
  static bool configured[PYLO_MAX_DEVICES] = {};
  constexpr int smem = (int)sizeof(NsSmem) + 1024;  // room to start the tiles on a 1024-byte boundary
  if (int rc = allow_dynamic_smem(k_gemm_tn_3xtf32, smem, configured)) return rc;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  k_gemm_tn_3xtf32<<<grid, NS_THREADS, smem, (cudaStream_t)stream>>>(a, status);
  return launch_status();
}

int pylo_b200_transpose(const float* src, float* dst, int rows, int cols, int ld_src, int ld_dst, int64_t stride_src,
                        int64_t stride_dst, int batch, int mirror, void* stream) {
  CHECK_ARG(src && dst && rows > 0 && cols > 0 && batch > 0 && batch <= 65535 && ld_src >= cols);
  if (mirror) CHECK_ARG(rows == cols && src == dst && ld_src == ld_dst);
  else CHECK_ARG(src != dst && ld_dst >= rows);
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  CHECK_ARG(grid.y <= 65535);
  k_transpose32<<<grid, 256, 0, (cudaStream_t)stream>>>(src, dst, rows, cols, ld_src, ld_dst, stride_src, stride_dst, mirror ? 1 : 0);
  return launch_status();
}

int pylo_b200_apply_packed(const pylo_tensor_desc* descs, const pylo_atile* ctiles, int n_ctiles,
                           const pylo_step_params* prm, void* stream) {
  CHECK_ARG(descs && ctiles && prm && n_ctiles >= 0);
  if (n_ctiles == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  switch (prm->family) {
    case PYLO_FAM_CELO2: k_apply_packed<PYLO_FAM_CELO2><<<grid_for(n_ctiles, 2), NT, 0, s>>>(descs, ctiles, n_ctiles, *prm); break;
    case PYLO_FAM_VELO: k_apply_packed<PYLO_FAM_VELO><<<grid_for(n_ctiles, PK_CTAS_VELO), NT, 0, s>>>(descs, ctiles, n_ctiles, *prm); break;
    default: return -2;
  }
  return launch_status();
}

int pylo_b200_celo2_post_sums(const pylo_post_item* items, const pylo_tile* tiles, int n_tiles, void* stream) {
  CHECK_ARG(items && tiles && n_tiles >= 0);
  if (n_tiles == 0) return 0;
  k_post_sums<<<grid_for(n_tiles, 8), NT, 0, (cudaStream_t)stream>>>(items, tiles, n_tiles);
  return launch_status();
}

int pylo_b200_celo2_post_apply(const pylo_post_item* items, const pylo_tile* tiles, int n_tiles, void* stream) {
  CHECK_ARG(items && tiles && n_tiles >= 0);
  if (n_tiles == 0) return 0;
  k_post_apply<<<grid_for(n_tiles, 8), NT, 0, (cudaStream_t)stream>>>(items, tiles, n_tiles);
  return launch_status();
}

int pylo_b200_adamw(const pylo_adam_item* items, const pylo_tile* tiles, int n_tiles, int independent, float beta1,
                    float one_minus_beta1, float beta2, float one_minus_beta2, float eps,
                    const pylo_step_params* prm, void* stream) {
  CHECK_ARG(items && tiles && prm && n_tiles >= 0);
  if (n_tiles == 0) return 0;
  k_adamw<<<grid_for(n_tiles, 8), NT, 0, (cudaStream_t)stream>>>(items, tiles, n_tiles, independent, beta1, one_minus_beta1, beta2,
                                                              one_minus_beta2, eps, *prm);
  return launch_status();
}

int pylo_b200_velo_tensor_features(const pylo_tensor_desc* descs, int n_local, const int32_t* layer_of,
                                   int n_total, const float* rank_onehot, const float* fraction9,
                                   const float* loss9, float* x_in, void* stream) {
  CHECK_ARG(descs && rank_onehot && fraction9 && loss9 && x_in && n_local > 0 && n_total >= n_local);
  k_velo_tensor_features<<<(n_local + 127) / 128, 128, 0, (cudaStream_t)stream>>>(descs, n_local, layer_of, n_total,
                                                                                 rank_onehot, fraction9, loss9, x_in);
  return launch_status();
}

int pylo_b200_velo_rnn(const pylo_velo_rnn* rnn, void* stream) {
  CHECK_ARG(rnn && rnn->T > 0 && rnn->H > 0 && rnn->B > 0 && rnn->B <= 1024);
  cudaStream_t s = (cudaStream_t)stream;
  const pylo_velo_rnn r = *rnn;
  const int64_t TH = (int64_t)r.T * r.H;
  k_velo_pool<<<(r.H + 127) / 128, 128, 0, s>>>(r);
  k_velo_xmix<<<(unsigned)((TH + 255) / 256), 256, 0, s>>>(r);
  k_velo_gates<<<dim3((4 * r.H + GT - 1) / GT, (r.T + GT - 1) / GT), NT, 0, s>>>(r);
  k_velo_cell<<<(unsigned)((TH + 255) / 256), 256, 0, s>>>(r);
  const int64_t hw = (int64_t)r.T * (r.B + 1);
  k_velo_heads<<<(unsigned)((hw + NWARP - 1) / NWARP), NT, 0, s>>>(r);
  k_velo_mix<<<r.T, 160, r.B * sizeof(float), s>>>(r);
  return launch_status();
}

int pylo_b200_velo_loss_features(float* means, int32_t* iteration, float* running_min, const float* decays,
                                 const float* loss, float* loss9, void* stream) {
  CHECK_ARG(means && iteration && running_min && decays && loss && loss9);
  k_velo_loss<<<1, 32, 0, (cudaStream_t)stream>>>(means, iteration, running_min, decays, loss, loss9);
  return launch_status();
}

}  // extern "C"
