// Phase C for AdafacLO / ELO on FAST2D tensors on the tensor cores with fp16 operands
// (`mlp_precision="2xfp16"`; included by pylo_kernels.cu after pylo_apply_tc.cuh, whose helpers it uses).
//
// Same organisation as k_apply_adafac_tc (a warpgroup = one 128-element tile, operand A in tensor
// memory, weights in shared memory, independent warpgroup workers), with these differences:
//   * every operand is split into an fp16 high part and an fp16 low part (11 + 11 significant bits,
//     the same as the TF32 split) and the products are kind::f16, which takes K = 16 per instruction:
//     13 products per tile instead of 25;
//   * two halves share a 32-bit tensor-memory column, so operand A takes 32 columns instead of 64
//     and six warpgroups fit an SM;
//   * fp16 has a narrow exponent range, so the features enter the product normalised: multiplied by
//     rsqrt(mean f^2 + eps), which the other kernels fold into the first-layer weights instead.  A
//     normalised feature is at most sqrt(n) < 65504 in magnitude for any tensor below 2^32 elements,
//     and a value far below its feature's rms keeps an absolute precision of 3e-8 of that rms.  The
//     conversions saturate, so a hidden activation beyond 65504 is clamped instead of turning inf.
#pragma once

#include <cuda_fp16.h>

#define TH_WGS 6
#define TH_NT (TH_WGS * 128)
#define TH_WG_TMEM 64            // tensor-memory columns per warpgroup: [0,16) A high, [16,32) A low, [32,64) accumulator
constexpr uint32_t TH_IDESC = (1u << 4) | ((32u >> 3) << 17) | ((128u >> 4) << 24);  // f16 x f16 -> f32, N = 32, M = 128

// index (in halves) of B[n][k] in the K-major no-swizzle layout: core matrices of 8 rows x 8 halves
__host__ __device__ constexpr int th_b_index(int n, int k) { return ((k >> 3) * TC_LBO + (n >> 3) * TC_SBO + (n & 7) * 16 + (k & 7) * 2) / 2; }

// D[128 x 32] (+)= A[128 x 16] * B[32 x 16]^T
__device__ __forceinline__ void th_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(TH_IDESC), "r"(accumulate) : "memory");
}
// (x0, x1) -> packed fp16 high parts and packed fp16 low parts; x0 goes to the low half (the even K index)
__device__ __forceinline__ void th_split(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(x1), "f"(x0));
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(x1 - f.y), "f"(x0 - f.x));
}
__device__ __forceinline__ void th_split1(float x, __half& hi, __half& lo) {
  hi = __float2half_rn(x);
  lo = __float2half_rn(x - __half2float(hi));
}

struct ThWgSmem {
  __half b1hi[32 * 32], b1lo[32 * 32];           // first layer: N = 32, K = 32 (28 features, bias row, 3 zero rows)
  __half b2hi[32 * 32], b2lo[32 * 32];           // second layer: N = 32, K = 32
  __half b2bias[32 * 16];                        // second-layer bias as a K = 16 block: (high part, low part, 0 ...)
  float w3[64 + 4];                              // output layer, pair-major (Fold::W3P), then its two biases
  float fscale[16];                              // normalisers of the 16 element-wise features
  float vscale[12];                              // normalisers of the row vector's six features, then the column vector's
  uint4 colf_a[TC_COLS];                         // the item's columns: three words of high parts, first word of low parts
  uint2 colf_b[TC_COLS];                         // ... the other two words of low parts
  uint4 rowf[2][3];                              // double-buffered row: 3 high words, 3 low words, the row's 3 factors, pad
  TcItem item;
  uint64_t bar;
};
struct ThSmem {
  ThWgSmem wg[TH_WGS];
  uint32_t tmem_base;
  int poisoned;  // the status word at launch: non-zero means an earlier launch reported a timed-out wait
};

// the pair (2c, 2c+1) of the six features of a vector entry: fac[0..2], then rsqrt(fac[0..2] + 1e-8)
__device__ __forceinline__ float th_vec6(float f0, float f1, float f2, int j) {
  const float r = j % 3 == 0 ? f0 : (j % 3 == 1 ? f1 : f2);
  return j < 3 ? r : rsqrtf(r + 1e-8f);
}

__global__ void __launch_bounds__(TH_NT, 1) k_apply_adafac_tc16(const pylo_tensor_desc* __restrict__ descs,
                                                                const pylo_atile* __restrict__ ttiles, int n_ttiles,
                                                                const pylo_step_params prm, int* __restrict__ status) {
  using F = Fam<PYLO_FAM_ADAFAC>;
  using L = Fold<PYLO_FAM_ADAFAC>;
  extern __shared__ __align__(128) unsigned char th_raw[];
  ThSmem& smem = *reinterpret_cast<ThSmem*>(th_raw);
  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, col = tid & 127;
  ThWgSmem& sm = smem.wg[wg];
  if (col == 0) mbar_init(&sm.bar, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (tid == 32) smem.poisoned = status ? *reinterpret_cast<volatile int*>(status) : 0;
  if (warp == 0) { tc_alloc(&smem.tmem_base, 512); tc_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // A launch that finds the status word already set writes nothing (no parameter, no peer store): the
  // parameters stay as the last good step left them until the host has looked at the error and cleared it.
  const int n_items = smem.poisoned ? 0 : n_ttiles;
  const uint32_t t_wg = smem.tmem_base + wg * TH_WG_TMEM;               // lane 0 of this warpgroup's columns
  const uint32_t t_lane = t_wg + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes
  const uint32_t tA = t_lane, tD = t_lane + 32;
  if (wg == 0) {  // the constant operand (1, 1, 0 ...) in halves: it adds the second-layer bias as one more product
    uint32_t one[8] = {0x3c003c00u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(smem.tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + TC_CONST_COL), "r"(one[0]), "r"(one[1]), "r"(one[2]),
                   "r"(one[3]), "r"(one[4]), "r"(one[5]), "r"(one[6]), "r"(one[7]) : "memory");
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();  // every warpgroup's products may read the constant operand
  tc_fence_after();
  constexpr uint64_t KSTEP = (2 * TC_LBO) >> 4;  // one product consumes two K chunks of 8 halves
  uint32_t parity = 0;
  bool timed_out = false;
  int loaded = -1;
  for (int t = blockIdx.x * TH_WGS + wg; t < n_items; t += gridDim.x * TH_WGS) {
    const pylo_atile ct = ttiles[t];
    const pylo_tensor_desc& d = descs[ct.tensor];
    const int X = d.X, Y = d.Y;
    const int rows_item = ct.pad_;
    const int y = ct.cb * TC_COLS + col;
    const bool colok = y < Y;
    const int yc = colok ? y : 0;
    const int x0 = ct.strip * rows_item;
    wg_barrier(wg);  // the four warps are done with the previous item's column terms and weights
    if (loaded != ct.tensor) {
      // K order of the first layer: 16 element-wise features (0..12, 25..27), the six features of the row vector,
      // the six of the column vector, the bias (against a constant 1), three zero rows.  Weights are the raw ones
      // (desc.w, [32][39]); the features' normalisers go to fscale / vscale.
      const int ka = d.r_is_a ? F::R : F::C, kra = d.r_is_a ? F::RR : F::RC;
      const int kb = d.r_is_a ? F::C : F::R, krb = d.r_is_a ? F::RC : F::RR;
      auto feature_of = [&](int kk) {
        return kk < 13 ? kk : kk < 16 ? kk + 12 : kk < 19 ? ka + kk - 16 : kk < 22 ? kra + kk - 19 : kk < 25 ? kb + kk - 22 : krb + kk - 25;
      };
      for (int e = col; e < 32 * 32; e += 128) {
        const int n = e & 31, kk = e >> 5;
        float w = 0.f;
        if (kk < 28) w = d.w[n * 39 + feature_of(kk)];
        else if (kk == 28) w = d.wfold[L::B1 + n];
        th_split1(w, sm.b1hi[th_b_index(n, kk)], sm.b1lo[th_b_index(n, kk)]);
      }
      for (int e = col; e < 32 * 32; e += 128) {
        const int n = e & 31, k = e >> 5;
        th_split1(d.wfold[L::W2 + k * 32 + n], sm.b2hi[th_b_index(n, k)], sm.b2lo[th_b_index(n, k)]);
      }
      for (int e = col; e < 32 * 16; e += 128) {
        const int n = e & 31, k = e >> 5;
        __half hi, lo;
        th_split1(d.wfold[L::B2 + n], hi, lo);
        sm.b2bias[th_b_index(n, k)] = k == 0 ? hi : (k == 1 ? lo : __float2half_rn(0.f));
      }
      if (col < 64) sm.w3[col] = d.wfold[L::W3P + col];
      if (col < 2) sm.w3[64 + col] = d.wfold[L::B3 + col];
      if (col < 28) {
        const float sc = rsqrtf(d.sums[feature_of(col)] / (float)d.n + prm.eps_norm);
        if (col < 16) sm.fscale[col] = sc;
        else sm.vscale[col - 16] = sc;
      }
      loaded = ct.tensor;
      wg_barrier(wg);  // vscale is read below
    }
    {  // this thread's column: six vector features, normalised and split, as three words of pairs each
      const float c0 = d.fac_b[yc], c1 = d.fac_b[(int64_t)Y + yc], c2 = d.fac_b[2 * (int64_t)Y + yc];
      uint32_t hi[3], lo[3];
#pragma unroll
      for (int q = 0; q < 3; ++q)
        th_split(colok ? th_vec6(c0, c1, c2, 2 * q) * sm.vscale[6 + 2 * q] : 0.f,
                 colok ? th_vec6(c0, c1, c2, 2 * q + 1) * sm.vscale[6 + 2 * q + 1] : 0.f, hi[q], lo[q]);
      sm.colf_a[col] = make_uint4(hi[0], hi[1], hi[2], lo[0]);
      sm.colf_b[col] = make_uint2(lo[1], lo[2]);
    }
    // row-wide values of the first row: threads 0..2 make one pair of the row vector's features each, 3..5 one factor
    auto put_row = [&](int buf, float f0, float f1, float f2, float fxv) {
      uint32_t* r = reinterpret_cast<uint32_t*>(&sm.rowf[buf][0]);
      if (col < 3) {
        uint32_t hi, lo;
        th_split(th_vec6(f0, f1, f2, 2 * col) * sm.vscale[2 * col], th_vec6(f0, f1, f2, 2 * col + 1) * sm.vscale[2 * col + 1], hi, lo);
        r[col] = hi;
        r[3 + col] = lo;
      } else if (col < 6) {
        r[6 + col - 3] = __float_as_uint(fxv);
      }
    };
    if (col < 6 && x0 < X)
      put_row(0, d.fac_a[x0], d.fac_a[(int64_t)X + x0], d.fac_a[2 * (int64_t)X + x0], d.fx[(int64_t)x0 * 4 + (col < 3 ? 0 : col - 3)]);
    if (col == 0) {
      TcItem& it = sm.item;
      it.g = d.g; it.p = d.p; it.m = d.m; it.v = d.v; it.fx = d.fx; it.fac_a = d.fac_a;
      it.peer = d.p_peer; it.n_peer = d.n_peer; it.n = d.n;
      it.exp_mult = d.exp_mult; it.step_mult = d.step_mult; it.wd = d.wd; it.lr = d.lr;
      it.lr_eff = d.wfold[L::SC + 1]; it.gs = grad_scale_of(d, prm); it.wd_mode = prm.wd_mode;
    }
    fence_async_smem();  // the tensor core reads the weights through the async proxy
    wg_barrier(wg);
    // column factors of the element-wise factored features, with those features' normalisers folded in
    const float fb0 = d.f_b[yc], fb1 = d.f_b[Y + yc], fb2 = d.f_b[2 * (int64_t)Y + yc];
    const volatile TcItem& ic = sm.item;
    // no clipping, no nan_to_num, no global-norm scale (AdafacLO's defaults): the gradient is used as it is
    const bool plain_grad = !prm.nan_to_num && prm.clip_val == CUDART_INF_F && ic.gs == 1.0f;
    float cg, cp, cm0, cm1, cm2, cv;
    auto load_row = [&](int x, float& g, float& p, float& m0, float& m1, float& m2, float& v) {
      const int64_t idx = (colok && x < X) ? (int64_t)x * Y + y : 0;
      const int64_t n = ic.n;
      const float* mp = ic.m;
      g = ldg_early(ic.g + idx); p = ldg_early(ic.p + idx); m0 = ldg_early(mp + idx);
      m1 = ldg_early(mp + n + idx); m2 = ldg_early(mp + 2 * n + idx); v = ldg_early(ic.v + idx);
    };
    load_row(x0, cg, cp, cm0, cm1, cm2, cv);
    // threads 0..5 carry the row-wide inputs of the row after next: the row vector's three factors (0..2, which
    // need all three for their pair) or one of the row's factors (3..5); global loads consumed an iteration later
    float nf0 = 1.f, nf1 = 1.f, nf2 = 1.f;
    auto load_next = [&](int x) {
      const int xs = x < X ? x : 0;
      if (col < 3) {
        nf0 = ldg_early(ic.fac_a + xs); nf1 = ldg_early(ic.fac_a + (int64_t)X + xs); nf2 = ldg_early(ic.fac_a + 2 * (int64_t)X + xs);
      } else if (col < 6) {
        nf0 = ldg_early(ic.fx + (int64_t)xs * 4 + (col - 3));
      }
    };
    load_next(x0 + 1);
#pragma unroll 1
    for (int i = 0; i < rows_item; ++i) {
      const int x = x0 + i;  // the same for the whole warpgroup
      if (x >= X) break;
      // the next row's row-wide values, for the next iteration (two warpgroup barriers lie in between)
      if (col < 6) put_row((i + 1) & 1, nf0, nf1, nf2, nf0);
      load_next(x + 2);
      // ---- operand A of the first layer: normalised features, high and low halves
      {
        const float g = plain_grad ? cg : xform_grad(cg, ic.gs, prm.clip_val, prm.nan_to_num);
        const float rs = rsqrt_pos(cv + prm.eps_feat);
        const uint4 rw0 = sm.rowf[i & 1][0], rw1 = sm.rowf[i & 1][1], rw2 = sm.rowf[i & 1][2];
        const float k0 = __uint_as_float(rw1.z) * fb0, k1 = __uint_as_float(rw1.w) * fb1, k2 = __uint_as_float(rw2.x) * fb2;
        const float4 s0 = *reinterpret_cast<const float4*>(&sm.fscale[0]), s1 = *reinterpret_cast<const float4*>(&sm.fscale[4]);
        const float4 s2 = *reinterpret_cast<const float4*>(&sm.fscale[8]), s3 = *reinterpret_cast<const float4*>(&sm.fscale[12]);
        const float fe[16] = {g * s0.x, cp * s0.y, cm0 * s0.z, cm1 * s0.w, cm2 * s1.x, cv * s1.y, cm0 * rs * s1.z, cm1 * rs * s1.w,
                              cm2 * rs * s2.x, rs * s2.y, k0 * g * s2.z, k1 * g * s2.w, k2 * g * s3.x, k0 * cm0 * s3.y,
                              k1 * cm1 * s3.z, k2 * cm2 * s3.w};
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int c = 0; c < 8; ++c) th_split(fe[2 * c], fe[2 * c + 1], hi[c], lo[c]);
        const uint4 ca = sm.colf_a[col];
        const uint2 cb = sm.colf_b[col];
        hi[8] = rw0.x; hi[9] = rw0.y; hi[10] = rw0.z; hi[11] = ca.x; hi[12] = ca.y; hi[13] = ca.z;
        hi[14] = 0x00003c00u;  // K slot 28 = 1 (the bias row), 29 = 0
        hi[15] = 0u;
        lo[8] = rw0.w; lo[9] = rw1.x; lo[10] = rw1.y; lo[11] = ca.w; lo[12] = cb.x; lo[13] = cb.y; lo[14] = 0u; lo[15] = 0u;
        tc_st16(tA, hi);
        tc_st16(tA + 16, lo);
      }
      // the next row's operands: requested now that this row's are consumed (only p is still needed)
      float np_;
      load_row(x + 1, cg, np_, cm0, cm1, cm2, cv);
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      if (col == 0) {
        tc_fence_after();
        const uint64_t desc_b1hi = tc_desc(smem_addr(sm.b1hi)), desc_b1lo = tc_desc(smem_addr(sm.b1lo));
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 16 + 8 * s, desc_b1hi + s * KSTEP, s > 0);  // lo x hi
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 8 * s, desc_b1lo + s * KSTEP, 1);           // hi x lo
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 8 * s, desc_b1hi + s * KSTEP, 1);           // hi x hi
        tc_commit(&sm.bar);
      }
      __syncwarp();
      if (!timed_out && !mbar_wait(&sm.bar, parity)) timed_out = true;
      parity ^= 1;
      tc_fence_after();
      // ---- hidden layer 1: relu, split into halves, back into tensor memory as operand A of the second layer
      {
        uint32_t dv0[16], dv1[16], hi[16], lo[16];
        tc_ld16(tD, dv0);
        tc_ld16(tD + 16, dv1);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          th_split(fmaxf(__uint_as_float(dv0[2 * c]), 0.f), fmaxf(__uint_as_float(dv0[2 * c + 1]), 0.f), hi[c], lo[c]);
          th_split(fmaxf(__uint_as_float(dv1[2 * c]), 0.f), fmaxf(__uint_as_float(dv1[2 * c + 1]), 0.f), hi[8 + c], lo[8 + c]);
        }
        tc_st16(tA, hi);
        tc_st16(tA + 16, lo);
      }
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      if (col == 0) {
        tc_fence_after();
        const uint64_t desc_b2hi = tc_desc(smem_addr(sm.b2hi)), desc_b2lo = tc_desc(smem_addr(sm.b2lo));
        th_mma(t_wg + 32, smem.tmem_base + TC_CONST_COL, tc_desc(smem_addr(sm.b2bias)), 0);               // bias
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 16 + 8 * s, desc_b2hi + s * KSTEP, 1);      // lo x hi
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 8 * s, desc_b2lo + s * KSTEP, 1);           // hi x lo
#pragma unroll
        for (int s = 0; s < 2; ++s) th_mma(t_wg + 32, t_wg + 8 * s, desc_b2hi + s * KSTEP, 1);           // hi x hi
        tc_commit(&sm.bar);
      }
      __syncwarp();
      if (!timed_out && !mbar_wait(&sm.bar, parity)) timed_out = true;
      parity ^= 1;
      tc_fence_after();
      // ---- hidden layer 2 (relu) and the two output heads as packed dot products over unit pairs
      uint64_t od[2] = {0ull, 0ull}, om[2] = {0ull, 0ull};
      {
        uint32_t dv0[16], dv1[16];
        tc_ld16(tD, dv0);
        tc_ld16(tD + 16, dv1);
        tc_wait_ld();
        auto heads = [&](const uint32_t (&dv)[16], int half) {
#pragma unroll
          for (int jp = 0; jp < 8; ++jp) {
            const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&sm.w3[4 * (half * 8 + jp)]);  // (dir pair, mag pair)
            const uint64_t r = pack2(fmaxf(__uint_as_float(dv[2 * jp]), 0.f), fmaxf(__uint_as_float(dv[2 * jp + 1]), 0.f));
            od[jp & 1] = fma2(w.x, r, od[jp & 1]);
            om[jp & 1] = fma2(w.y, r, om[jp & 1]);
          }
        };
        heads(dv0, 0);
        heads(dv1, 1);
      }
      {
        float a, b, c, dd;
        unpack2(add2(od[0], od[1]), a, b);
        unpack2(add2(om[0], om[1]), c, dd);
        const float o0 = (a + b) + sm.w3[64], o1 = (c + dd) + sm.w3[65];
        if (colok && !timed_out) {  // after a wait that ran out the accumulators are not to be trusted: keep the old value
          const Fin fin{ic.exp_mult, ic.step_mult, ic.wd, ic.lr, ic.lr_eff, 1.0f, ic.wd_mode};
          const float pn = finish<PYLO_FAM_ADAFAC>(cp, o0, o1, fin);
          const int64_t idx = (int64_t)x * Y + y;
          ic.p[idx] = pn;
          peer_store(Peers{ic.peer, ic.n_peer}, idx, pn);
        }
      }
      cp = np_;
    }
  }
  if (timed_out && status) atomicOr(status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(smem.tmem_base, 512);
}
