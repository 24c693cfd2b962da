// Phase C for AdafacLO / ELO on FAST2D tensors on the tensor cores (included by pylo_kernels.cu).
//
// The per-element network is a pair of small dense products, [elements x 29] x [29 x 32] and
// [elements x 32] x [32 x 32]; on the CUDA cores they cost ~1600 fp32 FMAs per element and bound the whole
// step.  Here a warpgroup (128 threads) treats 128 consecutive elements of one tensor row as the M = 128 rows
// of tcgen05 TF32 products:
//   * each thread builds its element's 16 element-wise features in registers and writes them with tcgen05.st
//     into tensor memory, where they are operand A (lane = element, column = feature);
//   * the six features that depend only on the element's column join operand A as six more columns, kept in
//     registers for all rows of a work item; the six that depend only on its ROW are the same for all 128
//     elements of the tile, so together with the first-layer bias they are a per-row bias vector: it is read from
//     the table k_prep_apply makes (desc.h_a, 32 floats per row) and enters the product through operand B, as two
//     rows (its high and low part) that meet two constant-1 columns of operand A.  First layer: K = 24;
//   * fp32 accuracy is kept by splitting every operand into a TF32 high part and a TF32 low part and running
//     three products per layer and K step (hi x hi, hi x lo, lo x hi) into one accumulator of 32 columns.  Operand
//     B holds the high parts in rows 0..31 and the low parts in rows 32..63 of one block; a product addresses
//     either half through its descriptor's start address.  A tile takes 9 + 13 = 22 products of width 32;
//   * the second-layer bias is one more product, of a constant operand A (ones, in shared memory) with a block of
//     operand B that holds the bias's high and low parts;
//   * relu, the split of the hidden activations, the two output heads and the parameter update stay on the CUDA
//     cores, which work on one warpgroup's tile while the tensor core works on another's: four warpgroups per
//     CTA (five fit), one CTA per SM; every warpgroup is an independent worker with its own work items, its own
//     copy of the weights in shared memory, its own 96 tensor-memory columns (32 operand A high parts, 32 low
//     parts, 32 accumulator) and its own barriers, so the warpgroups drift apart instead of marching in step;
//   * the products are issued by one elected lane inside a warp-uniform branch (the warp index is a broadcast
//     from lane 0), so that their descriptors and tensor-memory addresses live in uniform registers: issued from
//     a branch on the thread index, each product cost its thread ~52 cycles; this way ~24.
// Every wait on the tensor core is bounded.  A thread whose wait ran out records it in *status, stops waiting
// and stops storing (its parameters, and their copies on the peers, keep their old values), and goes on to
// the end, where the kernel frees its tensor memory.  A launch that finds *status already set stores nothing.
#pragma once

#ifndef TC_WGS
// Warpgroups per CTA (each uses 96 of the SM's 512 tensor-memory columns, so at most five).  Five are 8 % faster than
// four on a short run at the full clock (20.7 against 22.4 ps per element), but the full-size step runs at the GPU's
// power limit, where four win (246.7 against 250.3 ms per step, three: 262.4): four is the default.
#define TC_WGS 4
#endif
#define TC_NT (TC_WGS * 128)
#ifndef TC_BOUND_THREADS
#define TC_BOUND_THREADS TC_NT   // a larger bound lowers the register cap (65536 / bound): room for a co-resident kernel
#endif
#define TC_COLS 128              // tensor columns per work item: one per lane of the accumulator tile
#define TC_WG_TMEM 96            // tensor-memory columns per warpgroup: [0,32) operand A high parts, [32,64) low parts, [64,96) accumulator
#define TC_K1 24                 // first-layer K: 16 element-wise + 6 column features + 2 constant columns
#define TC_SPIN_LIMIT (1 << 20)
#ifndef TC_POLL_SLEEP_NS
#define TC_POLL_SLEEP_NS 40
#endif
#define TC_LBO 512               // bytes between 16-byte K chunks of a 32-row operand B (32 rows x 16 bytes)
#define TC_LBO64 1024            // the same for a 64-row operand B (high parts in rows 0..31, low parts in rows 32..63)
#define TC_LOW_HALF ((4 * TC_SBO) >> 4)   // descriptor start-address offset (16-byte units) of rows 32..63
#define TC_SBO 128               // bytes between groups of eight rows
#define TC_ONES_BYTES 2304       // constant operand A: every 16-byte chunk is (1, 1, 0, 0)

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
// one lane of the (converged) warp: true in exactly one thread
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void wg_barrier(int wg) { asm volatile("bar.sync %0, 128;" ::"r"(1 + wg) : "memory"); }

// D[128 x N] (+)= A[128 x 8] * B[N x 8]^T, A in tensor memory, B through a shared-memory descriptor
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with A through a shared-memory descriptor
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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

// 16 / 8 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}

// float index of B[n][k] in the K-major no-swizzle layout (8-row x 16-byte core matrices, K chunks `lbo` bytes apart)
__host__ __device__ constexpr int tc_b_index(int n, int k, int lbo = TC_LBO) {
  return ((k >> 2) * lbo + (n >> 3) * TC_SBO + (n & 7) * 16 + (k & 3) * 4) / 4;
}

// shared-memory matrix descriptor: start address, leading (K) and stride (row-group) byte offsets in 16-byte
// units, descriptor version 1, no swizzle
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr, int lbo = TC_LBO, int sbo = TC_SBO) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor: fp32 accumulate, TF32 x TF32, both operands K-major, M = 128, N = 32 or 64
__host__ __device__ constexpr uint32_t tc_idesc(uint32_t n) { return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
constexpr uint32_t TC_IDESC = tc_idesc(32);

// read-only 128-bit load issued where it is written (the compiler would otherwise sink it to its first use)
__device__ __forceinline__ float4 ldg4_early(const float* p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// Stage clocks (debug builds with -DTC_STAGE_CLOCKS only): lane 0 of every warpgroup's first warp adds the cycles it
// spends in each stage of a tile to status[8 + 12 * wg + stage].
#ifdef TC_STAGE_CLOCKS
#define TC_CLK_DECL long long clk_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long clk_t = clock64();
#define TC_CLK(stage) { const long long now_ = clock64(); clk_acc[stage] += now_ - clk_t; clk_t = now_; }
#define TC_CLK_FLUSH if (col == 0 && status) { for (int q_ = 0; q_ < 12; ++q_) atomicAdd(status + 8 + 12 * wg + q_, (int)(clk_acc[q_] >> 10)); }
#else
#define TC_CLK_DECL
#define TC_CLK(stage)
#define TC_CLK_FLUSH
#endif

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
// minus the TF32 high part of x: mask and sign flip are one three-input logic operation
__device__ __forceinline__ float tf32_hi_neg(float x) { return __uint_as_float((__float_as_uint(x) & 0xffffe000u) ^ 0x80000000u); }
// Split of 16 values for operand A.  hi: what goes into the high-part columns, lo: the low parts.
// The tensor core reads only the upper 19 bits of a TF32 operand (it truncates; the parity tests against the fp32
// kernel and the oracle would fail at the 1e-4 level if it rounded), so the high-part columns hold the unmasked
// value and the low parts are x + (-(x & mask)), two at a time with one packed add: 2.5 instructions per pair less
// than masking and subtracting (measured: 21.65 -> 20.65 ps per element).  -DTC_MASKED_HI builds the explicit form.
__device__ __forceinline__ void tc_split16(const float (&x)[16], uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#ifndef TC_MASKED_HI
#pragma unroll
  for (int k = 0; k < 16; k += 2) {
    float l0, l1;
    unpack2(add2(pack2(x[k], x[k + 1]), pack2(tf32_hi_neg(x[k]), tf32_hi_neg(x[k + 1]))), l0, l1);
    hi[k] = __float_as_uint(x[k]); hi[k + 1] = __float_as_uint(x[k + 1]);
    lo[k] = __float_as_uint(l0); lo[k + 1] = __float_as_uint(l1);
  }
#else
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float h = tf32_hi(x[k]);
    hi[k] = __float_as_uint(h);
    lo[k] = __float_as_uint(x[k] - h);
  }
#endif
}

// One warpgroup's private shared memory: its copy of the weights and its tensor-core barrier.  Warpgroups never
// wait on one another.
struct __align__(128) TcWgSmem {
  float b1[64 * TC_K1];   // first layer, rows 0..31 the high parts, 32..63 the low parts; K = 24 (K rows 22 and 23 of
                          // the high half are rewritten for every tensor row: the row's bias vector, high and low part)
  float b2[64 * 32];      // second layer, laid out the same way; K = 32
  float b2bias[32 * 8];   // second-layer bias as a K = 8 block: (high part, low part, 0 ...)
  float w3[64 + 4];       // output layer, pair-major (Fold::W3P), then its two biases
  uint64_t bar;
};
struct TcSmem {
  TcWgSmem wg[TC_WGS];
  __align__(128) float ones[TC_ONES_BYTES / 4];
  uint32_t tmem_base;
  int poisoned;  // the status word at launch: non-zero means an earlier launch reported a timed-out wait
};

__global__ void __launch_bounds__(TC_BOUND_THREADS, 1) k_apply_adafac_tc(const pylo_tensor_desc* __restrict__ descs,
                                                              const pylo_atile* __restrict__ ttiles, int n_ttiles,
                                                              const pylo_step_params prm, int* __restrict__ status) {
  using F = Fam<PYLO_FAM_ADAFAC>;
  using L = Fold<PYLO_FAM_ADAFAC>;
  extern __shared__ __align__(128) unsigned char tc_raw[];
  TcSmem& smem = *reinterpret_cast<TcSmem*>(tc_raw);
  const int tid = threadIdx.x, col = tid & 127;
  // The warp index as a value the compiler knows to be the same in all lanes (a broadcast from lane 0): the branch
  // that issues the products is then warp-uniform and its operands (descriptors, tensor-memory addresses) live in
  // uniform registers.  Issued from a branch on the thread index instead, a product cost its thread ~52 cycles on
  // top of the ~270 of the first; this way ~24 (6 products: 240 cycles instead of 522).
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0), wg = warp >> 2;
  TcWgSmem& sm = smem.wg[wg];
  if (col == 0) mbar_init(&sm.bar, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  for (int e = tid; e < TC_ONES_BYTES / 4; e += TC_NT) smem.ones[e] = (e & 3) < 2 ? 1.0f : 0.0f;
  if (tid == 32) smem.poisoned = status ? *reinterpret_cast<volatile int*>(status) : 0;
  if (warp == 0) { tc_alloc(&smem.tmem_base, 512); tc_relinquish(); }
  fence_async_smem();  // the constant operand is read by the tensor core through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // A launch that finds the status word already set writes nothing (no parameter, no peer store): the
  // parameters stay as the last good step left them until the host has looked at the error and cleared it.
  const int n_items = smem.poisoned ? 0 : n_ttiles;
  const uint32_t t_wg = __shfl_sync(0xffffffffu, smem.tmem_base, 0) + wg * TC_WG_TMEM;   // lane 0 of this warpgroup's columns
  const uint32_t t_lane = t_wg + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes
  const uint32_t tA = t_lane, tD = t_lane + 64;
  constexpr uint64_t KSTEP64 = (2 * TC_LBO64) >> 4;  // one product consumes two K chunks of operand B
  // every row of the constant operand is (1, 1, 0, 0, ...): any in-range chunk of the buffer holds that pattern
  const uint64_t desc_ones = tc_desc(smem_addr(smem.ones), 128, 128);
  uint32_t parity = 0;
  bool timed_out = false;
  int loaded = -1;
  TC_CLK_DECL
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
    wg_barrier(wg);  // the four warps are done with the previous item's weights
    if (loaded != ct.tensor) {
      // K order of the first layer: 16 element-wise features (0..12, 25..27), the six features of the column
      // vector, then the two rows that carry the tensor row's bias vector (written per row below)
      const int kb = d.r_is_a ? F::C : F::R, krb = d.r_is_a ? F::RC : F::RR;
      for (int e = col; e < 32 * TC_K1; e += 128) {
        const int n = e & 31, kk = e >> 5;
        float w = 0.f;
        if (kk < 13) w = d.wfold[L::W1 + kk * 32 + n];
        else if (kk < 16) w = d.wfold[L::W1 + (kk + 12) * 32 + n];
        else if (kk < 19) w = d.wfold[L::W1 + (kb + kk - 16) * 32 + n];
        else if (kk < 22) w = d.wfold[L::W1 + (krb + kk - 19) * 32 + n];
        const float hi = tf32_hi(w);
        sm.b1[tc_b_index(n, kk, TC_LBO64)] = hi;
        sm.b1[tc_b_index(32 + n, kk, TC_LBO64)] = w - hi;
      }
      for (int e = col; e < 32 * 32; e += 128) {
        const int n = e & 31, k = e >> 5;
        const float w = d.wfold[L::W2 + k * 32 + n], hi = tf32_hi(w);
        sm.b2[tc_b_index(n, k, TC_LBO64)] = hi;
        sm.b2[tc_b_index(32 + n, k, TC_LBO64)] = w - hi;
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
    // per-item constants: in registers for all rows of the item
    const float* __restrict__ gp = d.g;
    float* __restrict__ pp = d.p;
    const float* __restrict__ mp = d.m;
    const float* __restrict__ vp = d.v;
    const float* __restrict__ fxp = d.fx;    // [X][4]: the row's three factors of the element-wise factored features
    const float* __restrict__ hap = d.h_a;   // [X][32]: the row's first-layer bias vector (row features + bias)
    const int64_t n = d.n;
    const Peers peers = load_peers(d);
    const float gs = grad_scale_of(d, prm);
    const Fin fin{d.exp_mult, d.step_mult, d.wd, d.lr, d.wfold[L::SC + 1], 1.0f, prm.wd_mode};
    // no clipping, no nan_to_num, no global-norm scale (AdafacLO's defaults): the gradient is used as it is
    const bool plain_grad = !prm.nan_to_num && prm.clip_val == CUDART_INF_F && gs == 1.0f;
    const float fb0 = d.f_b[yc], fb1 = d.f_b[Y + yc], fb2 = d.f_b[2 * (int64_t)Y + yc];
    // the six features of this thread's column, high parts (then two ones) and low parts (then two zeros)
    uint32_t chi[8], clo[8];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      const float r = colok ? d.fac_b[(int64_t)(j % 3) * Y + yc] : 0.f;
      const float v = colok ? (j < 3 ? r : rsqrtf(r + 1e-8f)) : 0.f;
      const float hi = tf32_hi(v);
      chi[j] = __float_as_uint(hi);
      clo[j] = __float_as_uint(v - hi);
    }
    chi[6] = chi[7] = 0x3f800000u;
    clo[6] = clo[7] = 0u;
    fence_async_smem();  // the tensor core reads the weights through the async proxy
    wg_barrier(wg);
    float cg, cp, cm0, cm1, cm2, cv;
    float4 cfa;
    float hrow = 0.f;  // lanes 0..31 of the warpgroup's first warp: entry `col` of the row's bias vector
    auto load_row = [&](int x, float& g, float& p, float& m0, float& m1, float& m2, float& v, float4& fa, float& hr) {
      const int xc = x < X ? x : 0;
      const int64_t idx = (colok && x < X) ? (int64_t)x * Y + y : 0;
      g = ldg_early(gp + idx); p = ldg_early(pp + idx); m0 = ldg_early(mp + idx);
      m1 = ldg_early(mp + n + idx); m2 = ldg_early(mp + 2 * n + idx); v = ldg_early(vp + idx);
      fa = ldg4_early(fxp + 4 * (int64_t)xc);
      if (col < 32) hr = ldg_early(hap + (int64_t)xc * 32 + col);
    };
    load_row(x0, cg, cp, cm0, cm1, cm2, cv, cfa, hrow);
    TC_CLK(7)  // item set-up
#pragma unroll 1
    for (int i = 0; i < rows_item; ++i) {
      const int x = x0 + i;  // the same for the whole warpgroup
      if (x >= X) break;
      TC_CLK(8)  // loop overhead
      // ---- the row's bias vector into operand B (the previous row's first-layer products are complete)
      if (col < 32) {
        const float hi = tf32_hi(hrow);
        *reinterpret_cast<float2*>(&sm.b1[tc_b_index(col, 22, TC_LBO64)]) = make_float2(hi, hrow - hi);
        fence_async_smem();
      }
      TC_CLK(9)  // bias vector written
      // ---- operand A of the first layer, high and low parts
      {
        const float g = plain_grad ? cg : xform_grad(cg, gs, prm.clip_val, prm.nan_to_num);
        const float rs = rsqrt_pos(cv + prm.eps_feat);
        const float k0 = cfa.x * fb0, k1 = cfa.y * fb1, k2 = cfa.z * fb2;
        const float fe[16] = {g, cp, cm0, cm1, cm2, cv, cm0 * rs, cm1 * rs, cm2 * rs, rs,
                              k0 * g, k1 * g, k2 * g, k0 * cm0, k1 * cm1, k2 * cm2};
        uint32_t hi[16], lo[16];
        tc_split16(fe, hi, lo);
        TC_CLK(10)  // features and split
        tc_st16(tA, hi);
        tc_st8(tA + 16, chi);
        tc_st16(tA + 32, lo);
        tc_st8(tA + 48, clo);
      }
      // the next row's operands: requested now that this row's are consumed (only p is still needed, for the
      // update), so the two sets never share the register file; they land during the two products.  (Requesting
      // them at the top of the iteration instead, into registers of their own, measured 12 % slower.)
      float np_;
      load_row(x + 1, cg, np_, cm0, cm1, cm2, cv, cfa, hrow);
      TC_CLK(0)  // features, split, stores issued
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      TC_CLK(1)  // wait for the stores + warpgroup barrier
      if ((warp & 3) == 0) {
        if (elect_one()) {
          tc_fence_after();
          const uint64_t desc_b1 = tc_desc(smem_addr(sm.b1), TC_LBO64);
#pragma unroll
          for (int s = 0; s < 3; ++s) {
            tc_mma(t_wg + 64, t_wg + 32 + 8 * s, desc_b1 + s * KSTEP64, TC_IDESC, s > 0);          // lo x hi
            tc_mma(t_wg + 64, t_wg + 8 * s, desc_b1 + TC_LOW_HALF + s * KSTEP64, TC_IDESC, 1);     // hi x lo
          }
#pragma unroll
          for (int s = 0; s < 3; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b1 + s * KSTEP64, TC_IDESC, 1);   // hi x hi
          tc_commit(&sm.bar);
        }
        __syncwarp();
      }
      if (!timed_out && !mbar_wait(&sm.bar, parity)) timed_out = true;
      parity ^= 1;
      tc_fence_after();
      TC_CLK(2)  // first-layer products: issue + wait
      // ---- hidden layer 1: relu, split, back into tensor memory as operand A
      {
        uint32_t d0[16], d1[16];
        tc_ld16(tD, d0);        // everything is requested before anything is touched: one load latency
        tc_ld16(tD + 16, d1);
        tc_wait_ld();
        TC_CLK(3)  // accumulator read-back
        auto split_store = [&](const uint32_t (&a)[16], int half) {
          uint32_t hi[16], lo[16];
          float v[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) v[k] = fmaxf(__uint_as_float(a[k]), 0.f);
          tc_split16(v, hi, lo);
          tc_st16(tA + 16 * half, hi);
          tc_st16(tA + 32 + 16 * half, lo);
        };
        split_store(d0, 0);
        split_store(d1, 1);
      }
      TC_CLK(4)  // relu, split, stores issued
      tc_wait_st();
      tc_fence_before();
      wg_barrier(wg);
      TC_CLK(1)
      if ((warp & 3) == 0) {
        if (elect_one()) {
          tc_fence_after();
          const uint64_t desc_b2 = tc_desc(smem_addr(sm.b2), TC_LBO64);
          const uint64_t desc_b2bias = tc_desc(smem_addr(sm.b2bias));
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            tc_mma(t_wg + 64, t_wg + 32 + 8 * s, desc_b2 + s * KSTEP64, TC_IDESC, s > 0);          // lo x hi
            tc_mma(t_wg + 64, t_wg + 8 * s, desc_b2 + TC_LOW_HALF + s * KSTEP64, TC_IDESC, 1);     // hi x lo
          }
#pragma unroll
          for (int s = 0; s < 4; ++s) tc_mma(t_wg + 64, t_wg + 8 * s, desc_b2 + s * KSTEP64, TC_IDESC, 1);   // hi x hi
          tc_mma_ss(t_wg + 64, desc_ones, desc_b2bias, TC_IDESC, 1);                                         // bias
          tc_commit(&sm.bar);
        }
        __syncwarp();
      }
      if (!timed_out && !mbar_wait(&sm.bar, parity)) timed_out = true;
      parity ^= 1;
      tc_fence_after();
      TC_CLK(5)  // second-layer products: issue + wait
      // ---- hidden layer 2 (relu) and the two output heads as packed dot products over unit pairs
      uint64_t od[2] = {0ull, 0ull}, om[2] = {0ull, 0ull};
      {
        uint32_t d0[16], d1[16];
        tc_ld16(tD, d0);
        tc_ld16(tD + 16, d1);
        tc_wait_ld();
        TC_CLK(3)
        auto heads = [&](const uint32_t (&a)[16], int half) {
#pragma unroll
          for (int jp = 0; jp < 8; ++jp) {
            const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(&sm.w3[4 * (half * 8 + jp)]);  // (dir pair, mag pair)
            const uint64_t r = pack2(fmaxf(__uint_as_float(a[2 * jp]), 0.f), fmaxf(__uint_as_float(a[2 * jp + 1]), 0.f));
            od[jp & 1] = fma2(w.x, r, od[jp & 1]);
            om[jp & 1] = fma2(w.y, r, om[jp & 1]);
          }
        };
        heads(d0, 0);
        heads(d1, 1);
      }
      {
        float a, b, c, dd;
        unpack2(add2(od[0], od[1]), a, b);
        unpack2(add2(om[0], om[1]), c, dd);
        const float o0 = (a + b) + sm.w3[64], o1 = (c + dd) + sm.w3[65];
        if (colok && !timed_out) {  // after a wait that ran out the accumulators are not to be trusted: keep the old value
          const float pn = finish<PYLO_FAM_ADAFAC>(cp, o0, o1, fin);
          const int64_t idx = (int64_t)x * Y + y;
          pp[idx] = pn;
          peer_store(peers, idx, pn);
        }
      }
      cp = np_;
      TC_CLK(6)  // heads, update, store
    }
  }
  TC_CLK_FLUSH
  if (timed_out && status) atomicOr(status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(smem.tmem_base, 512);
}
