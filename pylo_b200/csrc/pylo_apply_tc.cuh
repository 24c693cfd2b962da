// Phase C for AdafacLO / ELO on FAST2D tensors, tensor-core variant (included by pylo_kernels.cu).
//
// The per-element network is a pair of small dense products, [elements x 29] x [29 x 32] and
// [elements x 32] x [32 x 32]; on the CUDA cores they cost ~1600 fp32 FMAs per element and bound
// the whole step.  Here a warpgroup (128 threads) treats 128 consecutive elements of one tensor
// row as the M = 128 rows of a tcgen05 TF32 product:
//   * each thread builds its element's 16 element-wise features in registers and writes them with
//     tcgen05.st into tensor memory, where they are operand A (lane = element, column = feature);
//   * the twelve features that depend only on the row or only on the column join operand A as
//     further columns (their split is made once per row by a few threads and once per work item
//     per column), the first-layer bias rides on a constant-1 column, and the second-layer bias
//     on one more small product against a constant operand;
//   * fp32 accuracy is kept by splitting every operand into a TF32 high part and a TF32 low part
//     and issuing three products per layer (lo x hi, hi x lo, hi x hi): the error of a 32-term dot
//     product is ~3e-7 of the sum of its terms' magnitudes, against ~1.5e-7 for an fp32 FMA chain;
//   * the weights (operand B) sit in shared memory in the K-major no-swizzle core-matrix layout,
//     split the same way, rebuilt only when the CTA moves to another tensor;
//   * relu, the split of the hidden activations, the two output heads and the parameter update
//     stay on the CUDA cores, which work on one warpgroup's tile while the tensor core works on
//     another's: five warpgroups per CTA, one CTA per SM; every warpgroup is an independent worker
//     with its own work items, its own copy of the weights in shared memory, its own accumulator
//     columns and its own barriers, so the warpgroups drift apart instead of marching in step.
// Every wait on the tensor core is bounded.  A thread whose wait ran out records it in *status, stops waiting
// and stops storing (its parameters, and their copies on the peers, keep their old values), and goes on to
// the end, where the kernel frees its tensor memory.  A launch that finds *status already set stores nothing.
#pragma once

#ifndef TC_WGS
#define TC_WGS 5                 // warpgroups per CTA: 5 x 96 tensor-memory columns + 8 shared ones fit the SM's 512
#endif
#define TC_NT (TC_WGS * 128)
#define TC_COLS 128              // tensor columns per work item: one per lane of the accumulator tile
#define TC_WG_TMEM 96            // tensor-memory columns per warpgroup: [0,64) operand A, [64,96) accumulator
#define TC_CONST_COL 480         // columns [480,488): the constant operand (1, 1, 0 ...) shared by all warpgroups
#define TC_SPIN_LIMIT (1 << 20)
#ifndef TC_POLL_SLEEP_NS
#define TC_POLL_SLEEP_NS 40
#endif
#define TC_LBO 512               // bytes between 16-byte K chunks of operand B (32 rows x 16 bytes)
#define TC_SBO 128               // bytes between groups of eight rows of operand B

__device__ __forceinline__ void tc_alloc(uint32_t* dst_smem, int ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, int ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void wg_barrier(int wg) { asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory"); }

// D[128 x 32] (+)= A[128 x 8] * B[32 x 8]^T, A in tensor memory, B through a shared-memory descriptor
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
// bounded wait for the phase with the given parity to complete; false on timeout
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  for (int it = 0; it < TC_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
    __nanosleep(TC_POLL_SLEEP_NS);  // back off: a waiting warp should not spend the issue slots of the working ones
  }
  return false;
}

// 16 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}

// float index of B[n][k] in the K-major no-swizzle layout: 8 x 16-byte core matrices, K chunks TC_LBO apart
__host__ __device__ constexpr int tc_b_index(int n, int k) { return ((k >> 2) * TC_LBO + (n >> 3) * TC_SBO + (n & 7) * 16 + (k & 3) * 4) / 4; }

// shared-memory matrix descriptor: start address, leading (K) and stride (row-group) byte offsets in 16-byte
// units, descriptor version 1, no swizzle
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(TC_LBO >> 4) << 16) | ((uint64_t)(TC_SBO >> 4) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor: fp32 accumulate, TF32 x TF32, both operands K-major, N = 32, M = 128
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);

// read-only 128-bit load issued where it is written (the compiler would otherwise sink it to its first use)
__device__ __forceinline__ float4 ldg4_early(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// per-item constants; they are read back from shared memory at their points of use (volatile, so that the
// compiler does not hoist them into registers for the whole row loop: at 512 threads a thread has 128 registers)
struct TcItem {
  const float* g;
  float* p;
  const float* m;
  const float* v;
  const float* fx;
  const float* fac_a;
  float* const* peer;
  long long n;
  float exp_mult, step_mult, wd, lr, lr_eff, gs;
  int wd_mode, n_peer;
};

// One warpgroup's private shared memory: its copy of the weights, the vector features of its item's columns and
// of its row in flight, its item constants and its tensor-core barrier.  Warpgroups never wait on one another.
struct TcWgSmem {
  float b1hi[32 * 32], b1lo[32 * 32];            // first layer: N = 32, K = 32 (28 features, bias row, 3 zero rows)
  float b2hi[32 * 32], b2lo[32 * 32];            // second layer: N = 32, K = 32
  float b2bias[32 * 8];                          // second-layer bias as a K = 8 block: (high part, low part, 0 ...)
  float w3[64 + 4];                              // output layer, pair-major (Fold::W3P), then its two biases
  float4 colf[3][TC_COLS];                       // the item's columns: 6 vector features, high parts then low parts
  float4 rowf[2][4];                             // double-buffered: the same for the row in flight / the next, then the
                                                 // row's three factors of the element-wise factored features
  TcItem item;
  uint64_t bar;
};
struct TcSmem {
  TcWgSmem wg[TC_WGS];
  uint32_t tmem_base;
  int poisoned;  // the status word at launch: non-zero means an earlier launch reported a timed-out wait
};

// the six vector features of one index of the "a" or "b" vector, feature j of 6: fac[j] (j < 3) or rsqrt(fac[j-3] + 1e-8)
__device__ __forceinline__ float tc_vec_feature(const float* __restrict__ fac, int64_t len, int64_t i, int j) {
  const float r = fac[(int64_t)(j % 3) * len + i];
  return j < 3 ? r : rsqrtf(r + 1e-8f);
}
// slot of feature j (0..5) in the three float4 of high and low parts
__device__ __forceinline__ void tc_put6(float4* q, int j, float v) {
  const float hi = tf32_hi(v);
  reinterpret_cast<float*>(q)[j] = hi;
  reinterpret_cast<float*>(q)[6 + j] = v - hi;
}

__global__ void __launch_bounds__(TC_NT, 1) k_apply_adafac_tc(const pylo_tensor_desc* __restrict__ descs,
                                                              const pylo_atile* __restrict__ ttiles, int n_ttiles,
                                                              const pylo_step_params prm, int* __restrict__ status) {
  using F = Fam<PYLO_FAM_ADAFAC>;
  using L = Fold<PYLO_FAM_ADAFAC>;
  extern __shared__ __align__(128) unsigned char tc_raw[];
  TcSmem& smem = *reinterpret_cast<TcSmem*>(tc_raw);
  const int tid = threadIdx.x, warp = tid >> 5, wg = tid >> 7, col = tid & 127;
  TcWgSmem& sm = smem.wg[wg];
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
  const uint32_t t_wg = smem.tmem_base + wg * TC_WG_TMEM;               // lane 0 of this warpgroup's columns
  const uint32_t t_lane = t_wg + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes
  const uint32_t tA = t_lane, tD = t_lane + 64;
  if (wg == 0) {  // the constant operand (1, 1, 0 ...) that adds the second-layer bias as one more product
    uint32_t one[8] = {0x3f800000u, 0x3f800000u, 0u, 0u, 0u, 0u, 0u, 0u};
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(smem.tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + TC_CONST_COL), "r"(one[0]), "r"(one[1]), "r"(one[2]),
                   "r"(one[3]), "r"(one[4]), "r"(one[5]), "r"(one[6]), "r"(one[7]) : "memory");
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();  // every warpgroup's products may read the constant operand
  tc_fence_after();
  constexpr uint64_t KSTEP = (2 * TC_LBO) >> 4;  // one product consumes two K chunks
  uint32_t parity = 0;
  bool timed_out = false;
  int loaded = -1;
  // every warpgroup is a worker of its own: it takes every (gridDim.x * TC_WGS)-th work item
  for (int t = blockIdx.x * TC_WGS + wg; t < n_items; t += gridDim.x * TC_WGS) {
    const pylo_atile ct = ttiles[t];
    const pylo_tensor_desc& d = descs[ct.tensor];
    const int X = d.X, Y = d.Y;
    const int rows_item = ct.pad_;  // rows per work item
    const int y = ct.cb * TC_COLS + col;
    const bool colok = y < Y;
    const int yc = colok ? y : 0;
    const int x0 = ct.strip * rows_item;
    wg_barrier(wg);  // the four warps are done with the previous item's column terms and weights
    if (loaded != ct.tensor) {
      // K order of the first layer: 16 element-wise features (0..12, 25..27), the six features of the row vector,
      // the six of the column vector, the bias (against a constant 1), three zero rows
      const int ka = d.r_is_a ? F::R : F::C, kra = d.r_is_a ? F::RR : F::RC;
      const int kb = d.r_is_a ? F::C : F::R, krb = d.r_is_a ? F::RC : F::RR;
      for (int e = col; e < 32 * 32; e += 128) {
        const int n = e & 31, kk = e >> 5;
        float w = 0.f;
        if (kk < 13) w = d.wfold[L::W1 + kk * 32 + n];
        else if (kk < 16) w = d.wfold[L::W1 + (kk + 12) * 32 + n];
        else if (kk < 19) w = d.wfold[L::W1 + (ka + kk - 16) * 32 + n];
        else if (kk < 22) w = d.wfold[L::W1 + (kra + kk - 19) * 32 + n];
        else if (kk < 25) w = d.wfold[L::W1 + (kb + kk - 22) * 32 + n];
        else if (kk < 28) w = d.wfold[L::W1 + (krb + kk - 25) * 32 + n];
        else if (kk == 28) w = d.wfold[L::B1 + n];
        const float hi = tf32_hi(w);
        sm.b1hi[tc_b_index(n, kk)] = hi;
        sm.b1lo[tc_b_index(n, kk)] = w - hi;
      }
      for (int e = col; e < 32 * 32; e += 128) {
        const int n = e & 31, k = e >> 5;
        const float w = d.wfold[L::W2 + k * 32 + n], hi = tf32_hi(w);
        sm.b2hi[tc_b_index(n, k)] = hi;
        sm.b2lo[tc_b_index(n, k)] = w - hi;
      }
      for (int e = col; e < 32 * 8; e += 128) {
        const int n = e & 31, k = e >> 5;
        const float w = d.wfold[L::B2 + n], hi = tf32_hi(w);
        sm.b2bias[tc_b_index(n, k)] = k == 0 ? hi : (k == 1 ? w - hi : 0.f);
      }
      if (col < 64) sm.w3[col] = d.wfold[L::W3P + col];
      if (col < 2) sm.w3[64 + col] = d.wfold[L::B3 + col];
      loaded = ct.tensor;
    }
    for (int e = col; e < 6 * TC_COLS; e += 128) {
      const int j = e / TC_COLS, c = e % TC_COLS, yy = ct.cb * TC_COLS + c;
      const float v = yy < Y ? tc_vec_feature(d.fac_b, Y, yy, j) : 0.f;
      const float hi = tf32_hi(v);
      reinterpret_cast<float*>(&sm.colf[j >> 2][c])[j & 3] = hi;
      reinterpret_cast<float*>(&sm.colf[(6 + j) >> 2][c])[(6 + j) & 3] = v - hi;
    }
    if (col < 6 && x0 < X) tc_put6(&sm.rowf[0][0], col, tc_vec_feature(d.fac_a, X, x0, col));
    if (col >= 6 && col < 9 && x0 < X) reinterpret_cast<float*>(&sm.rowf[0][3])[col - 6] = d.fx[(int64_t)x0 * 4 + (col - 6)];
    if (col == 0) {
      TcItem& it = sm.item;
      it.g = d.g; it.p = d.p; it.m = d.m; it.v = d.v; it.fx = d.fx; it.fac_a = d.fac_a;
      it.peer = d.p_peer; it.n_peer = d.n_peer; it.n = d.n;
      it.exp_mult = d.exp_mult; it.step_mult = d.step_mult; it.wd = d.wd; it.lr = d.lr;
      it.lr_eff = d.wfold[L::SC + 1]; it.gs = grad_scale_of(d, prm); it.wd_mode = prm.wd_mode;
    }
    fence_async_smem();  // the tensor core reads the weights through the async proxy
    wg_barrier(wg);
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
    // threads 0..8 carry one row-wide value for the row after next: the row vector's factor (0..5) or one of the
    // row's three factors (6..8); one global load each, consumed an iteration later, so that its latency never sits
    // between two barriers
    auto load_fac = [&](int x) {
      const float* src = ic.fac_a;
      int64_t off = 0;
      if (x < X) {
        if (col < 6) off = (int64_t)(col % 3) * X + x;
        else if (col < 9) { src = ic.fx; off = (int64_t)x * 4 + (col - 6); }
      }
      return ldg_early(src + off);
    };
    float fac_next = load_fac(x0 + 1);
#pragma unroll 1
    for (int i = 0; i < rows_item; ++i) {
      const int x = x0 + i;  // the same for the whole warpgroup
      if (x >= X) break;
      // the next row's row-wide values, for the next iteration (two warpgroup barriers lie in between)
      if (col < 6) tc_put6(&sm.rowf[(i + 1) & 1][0], col, col < 3 ? fac_next : rsqrtf(fac_next + 1e-8f));
      else if (col < 9) reinterpret_cast<float*>(&sm.rowf[(i + 1) & 1][3])[col - 6] = fac_next;
      fac_next = load_fac(x + 2);
      // ---- operand A of the first layer, high and low parts
      {
        const float g = plain_grad ? cg : xform_grad(cg, ic.gs, prm.clip_val, prm.nan_to_num);
        const float rs = rsqrt_pos(cv + prm.eps_feat);
        const float4 cfa = sm.rowf[i & 1][3];
        const float k0 = cfa.x * fb0, k1 = cfa.y * fb1, k2 = cfa.z * fb2;
        const float fe[16] = {g, cp, cm0, cm1, cm2, cv, cm0 * rs, cm1 * rs, cm2 * rs, rs,
                              k0 * g, k1 * g, k2 * g, k0 * cm0, k1 * cm1, k2 * cm2};
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float h = tf32_hi(fe[k]);
          hi[k] = __float_as_uint(h);
          lo[k] = __float_as_uint(fe[k] - h);
        }
        tc_st16(tA, hi);
        tc_st16(tA + 32, lo);
        const float4 r0 = sm.rowf[i & 1][0], r1 = sm.rowf[i & 1][1], r2 = sm.rowf[i & 1][2];
        const float4 c0 = sm.colf[0][col], c1 = sm.colf[1][col], c2 = sm.colf[2][col];
        // (r0, r1.xy) = row high parts, (r1.zw, r2) = row low parts; the same for the column
        const uint32_t vhi[16] = {__float_as_uint(r0.x), __float_as_uint(r0.y), __float_as_uint(r0.z), __float_as_uint(r0.w),
                                  __float_as_uint(r1.x), __float_as_uint(r1.y), __float_as_uint(c0.x), __float_as_uint(c0.y),
                                  __float_as_uint(c0.z), __float_as_uint(c0.w), __float_as_uint(c1.x), __float_as_uint(c1.y),
                                  0x3f800000u, 0u, 0u, 0u};
        const uint32_t vlo[16] = {__float_as_uint(r1.z), __float_as_uint(r1.w), __float_as_uint(r2.x), __float_as_uint(r2.y),
                                  __float_as_uint(r2.z), __float_as_uint(r2.w), __float_as_uint(c1.z), __float_as_uint(c1.w),
                                  __float_as_uint(c2.x), __float_as_uint(c2.y), __float_as_uint(c2.z), __float_as_uint(c2.w),
                                  0u, 0u, 0u, 0u};
        tc_st16(tA + 16, vhi);
        tc_st16(tA + 48, vlo);
      }
      // the next row's operands: requested now that this row's are consumed (only p is still needed, for the
      // update), so the two sets never share the register file; they land during the two products
      float np_;
      load_row(x + 1, cg, np_, cm0, cm1, cm2, cv);
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      if (col == 0) {
        tc_fence_after();
        const uint64_t desc_b1hi = tc_desc(smem_addr(sm.b1hi)), desc_b1lo = tc_desc(smem_addr(sm.b1lo));
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 32 + 8 * s, desc_b1hi + s * KSTEP, TC_IDESC, s > 0);  // lo x hi
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b1lo + s * KSTEP, TC_IDESC, 1);           // hi x lo
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b1hi + s * KSTEP, TC_IDESC, 1);           // hi x hi
        tc_commit(&sm.bar);
      }
      __syncwarp();
      if (!timed_out && !mbar_wait(&sm.bar, parity)) timed_out = true;
      parity ^= 1;
      tc_fence_after();
      // ---- hidden layer 1: relu, split, back into tensor memory as operand A of the second layer
      {
        uint32_t dv0[16], dv1[16];
        tc_ld16(tD, dv0);       // both halves are requested before the first is touched: one load latency, not two
        tc_ld16(tD + 16, dv1);
        tc_wait_ld();
        auto split_store = [&](const uint32_t (&dv)[16], int half) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float h = fmaxf(__uint_as_float(dv[k]), 0.f), hh = tf32_hi(h);
            hi[k] = __float_as_uint(hh);
            lo[k] = __float_as_uint(h - hh);
          }
          tc_st16(tA + 16 * half, hi);
          tc_st16(tA + 32 + 16 * half, lo);
        };
        split_store(dv0, 0);
        split_store(dv1, 1);
      }
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      if (col == 0) {
        tc_fence_after();
        const uint64_t desc_b2hi = tc_desc(smem_addr(sm.b2hi)), desc_b2lo = tc_desc(smem_addr(sm.b2lo));
        const uint64_t desc_b2bias = tc_desc(smem_addr(sm.b2bias));
        tc_mma(t_wg + 64, smem.tmem_base + TC_CONST_COL, desc_b2bias, TC_IDESC, 0);                                // bias
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 32 + 8 * s, desc_b2hi + s * KSTEP, TC_IDESC, 1);      // lo x hi
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b2lo + s * KSTEP, TC_IDESC, 1);           // hi x lo
#pragma unroll
        for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b2hi + s * KSTEP, TC_IDESC, 1);           // hi x hi
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
