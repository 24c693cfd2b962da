// fp32-faithful batched matrix product on the tensor cores, for the Newton-Schulz iteration of the CELO2 family
// (included by pylo_kernels.cu after pylo_apply_tc.cuh, whose tcgen05 helpers it uses).
//
//   C[b][m][n] = alpha * sum_k A[b][m][k] * B[b][n][k]  +  beta * D[b][m][n]          (both operands K-major)
//
// The three products of one Newton-Schulz round (CELO2_naive.py:59-73: a = x x^T, b = c1 a + c2 a a, x = c0 x + b x)
// all have this form once x^T is kept beside x (a is symmetric, so a a = a a^T), with the scaled additions as the
// epilogue.  The operands are plain fp32 matrices; fp32 accuracy comes from splitting every operand element into a
// TF32 high part (x rounded to nearest) and a low part (the exact remainder) and accumulating lo x hi, hi x lo and
// hi x hi in the fp32 accumulator, small terms first.
//
// symmetric != 0 (M = N, the result is known to be symmetric, as x x^T and a a are): only the tiles that reach the
// diagonal or lie above it are computed; the part below the diagonal is left untouched for k_mirror_lower.
//
// The tensor core adds into its fp32 accumulator with truncation, so a long accumulation drifts (measured: 3e-6 of
// sum |a||b| after K = 3072 against 3e-7 for an fp32 FMA chain).  The contraction is therefore cut into chunks of
// 256: each chunk is accumulated in tensor memory from zero, and the chunks are added up by the CUDA cores with
// round-to-nearest into a running sum that lives in the other half of tensor memory.
//
// One persistent CTA per SM, 21 warps in three roles:
//   * 16 loader warps in two groups; group g fills shared-memory stage g with every second K block of 32: 128-bit
//     global loads into registers (four full 128-byte rows per warp instruction; issued before the wait for the
//     stage to be free, so they are in flight while the other stage is being multiplied), the split on the CUDA
//     cores, 128-bit stores of the high and the low tile in the K-major 128-byte-swizzle layout the tensor core
//     reads at full rate (a row is 128 bytes, its 16-byte pieces XOR-ed with the row index modulo 8; both the
//     stores and the operand fetches are conflict-free), then a proxy fence and an arrive on the stage's "full"
//     barrier;
//   * one issuing thread: per K block it waits for "full", issues 12 tcgen05.mma (three products x four K steps of
//     8; M = 128, N = 256, A and B through shared-memory descriptors) into the 256-column chunk accumulator, and
//     commits to the stage's "empty" barrier; after the last K block of a chunk it commits to "chunk ready";
//   * four epilogue warps (one thread per accumulator lane = output row): after every chunk they add the chunk
//     accumulator into the running sum (tcgen05.ld / add / tcgen05.st, 32 columns at a time) and release it; after a
//     tile's last chunk they scale, add beta * D and store C with 128-bit stores instead.
// No TMA and no cluster features: the kernel runs unchanged inside a multi-GPU step.  Every wait is bounded; a
// wait that runs out raises a CTA-wide abort flag, every role leaves its loops, *status gets bit 2, and the
// tensor memory is freed.
#pragma once

#define NS_BM 128
#define NS_BN 256
#define NS_BK 32
#define NS_EPI_WARPS 4
#define NS_LOADER_WARPS 16
#define NS_THREADS ((NS_EPI_WARPS + 1 + NS_LOADER_WARPS) * 32)
#define NS_KCHUNK_BLOCKS 8      // K blocks per accumulation chunk (256 terms)
#define NS_SPIN_LIMIT (1 << 22)

struct NsStage {
  float a_hi[NS_BM * NS_BK], a_lo[NS_BM * NS_BK];
  float b_hi[NS_BN * NS_BK], b_lo[NS_BN * NS_BK];
};
struct NsSmem {
  NsStage st[2];   // every tile starts on a 1024-byte boundary (the swizzle pattern repeats every 8 rows of 128 bytes)
  uint64_t full[2], empty[2], chunk_ready, chunk_free;
  uint32_t tmem_base;
  volatile int abort;
};

// byte offset of the 16-byte piece `chunk` (0..7) of row `row` in a K-major tile with 128-byte rows and 128-byte swizzle
__device__ __forceinline__ int ns_swz(int row, int chunk) { return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4); }
// descriptor of such a tile: 8-row groups 1024 bytes apart, swizzle mode 2 (128 bytes), descriptor version 1
__device__ __forceinline__ uint64_t ns_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}

// x rounded to the nearest TF32 value (10 explicit mantissa bits), as an fp32 number
__device__ __forceinline__ float tf32_rn(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

struct pylo_gemm_args {  // mirrors pylo_gemm_desc (passed by value)
  const float* A; const float* B; float* C; const float* D;
  long long sA, sB, sC, sD;   // batch strides in floats
  int M, N, K, lda, ldb, ldc, ldd, batch;
  float alpha, beta;
  int symmetric, pad_;
};

// Tiles of one matrix in the order they are taken: all of them, or (symmetric) for every row of tiles only those
// whose 256 columns are not entirely below the diagonal of its 128 rows, i.e. tn >= tm / 2.
__host__ __device__ inline int ns_tiles_per_matrix(int tiles_m, int tiles_n, int symmetric) {
  if (!symmetric) return tiles_m * tiles_n;
  int n = 0;
  for (int tm = 0; tm < tiles_m; ++tm) n += tiles_n > tm / 2 ? tiles_n - tm / 2 : 0;
  return n;
}
__device__ __forceinline__ void ns_tile_coords(int r, int tiles_m, int tiles_n, int symmetric, int& tm, int& tn) {
  if (!symmetric) { tm = r / tiles_n; tn = r % tiles_n; return; }
  for (tm = 0; tm < tiles_m; ++tm) {
    const int cnt = tiles_n > tm / 2 ? tiles_n - tm / 2 : 0;
    if (r < cnt) { tn = tm / 2 + r; return; }
    r -= cnt;
  }
  tm = 0; tn = 0;
}

__device__ __forceinline__ bool ns_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  const uint32_t a = smem_addr(bar);
  for (int it = 0; it < NS_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
    if ((it & 63) == 63 && *abort) return false;
  }
  *abort = 1;
  return false;
}
__device__ __forceinline__ void ns_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(NS_THREADS, 1) k_gemm_tn_3xtf32(const pylo_gemm_args g, int* __restrict__ status) {
  extern __shared__ unsigned char ns_raw[];
  // the tiles need 1024-byte alignment; dynamic shared memory only promises 16
  NsSmem& sm = *reinterpret_cast<NsSmem*>(ns_raw + ((1024 - (smem_addr(ns_raw) & 1023)) & 1023));
  // the warp index as a broadcast from lane 0: the compiler then knows the role branches to be warp-uniform, and
  // the issuing branch keeps its descriptors and tensor-memory addresses in uniform registers
  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  if (tid == 0) {
    // full: one arrive per loader warp of the stage's group; empty and chunk_ready: one tcgen05.commit;
    // chunk_free: one arrive per epilogue warp
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.full[s], NS_LOADER_WARPS / 2);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.chunk_ready, 1);
    mbar_init(&sm.chunk_free, NS_EPI_WARPS);
    sm.abort = 0;
  }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (warp == NS_EPI_WARPS) { tc_alloc(&sm.tmem_base, 512); tc_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, sm.tmem_base, 0);   // columns [0,256): chunk accumulator, [256,512): running sum
  const int tiles_m = (g.M + NS_BM - 1) / NS_BM, tiles_n = (g.N + NS_BN - 1) / NS_BN;
  const int tiles_per_batch = ns_tiles_per_matrix(tiles_m, tiles_n, g.symmetric);
  const long long n_tiles = (long long)tiles_per_batch * g.batch;
  const int n_kb = (g.K + NS_BK - 1) / NS_BK;
  const int n_chunks = (n_kb + NS_KCHUNK_BLOCKS - 1) / NS_KCHUNK_BLOCKS;

  if (warp < NS_EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue: one thread per output row
    long long cc = 0;  // chunks seen so far
    const uint32_t t_acc = tmem + ((uint32_t)(warp * 32) << 16), t_run = t_acc + NS_BN;
    bool dead = false;
    for (long long tile = blockIdx.x; tile < n_tiles && !dead && !sm.abort; tile += gridDim.x) {
      const int b = (int)(tile / tiles_per_batch), r = (int)(tile % tiles_per_batch);
      int tm, tn;
      ns_tile_coords(r, tiles_m, tiles_n, g.symmetric, tm, tn);
      const int m = tm * NS_BM + warp * 32 + lane;
      const bool row_ok = m < g.M;
      float* crow = g.C + (long long)b * g.sC + (long long)(row_ok ? m : 0) * g.ldc;
      const float* drow = g.D ? g.D + (long long)b * g.sD + (long long)(row_ok ? m : 0) * g.ldd : nullptr;
      for (int c = 0; c < n_chunks; ++c, ++cc) {
        if (!ns_wait(&sm.chunk_ready, (uint32_t)(cc & 1), &sm.abort)) { dead = true; break; }
        tc_fence_after();
        const bool last = c == n_chunks - 1;
#pragma unroll 1
        for (int c0 = 0; c0 < NS_BN; c0 += 32) {
          uint32_t v[32];
          tc_ld32(t_acc + c0, v);
          if (c > 0) {  // add the running sum (round to nearest, on the CUDA cores)
            uint32_t w[32];
            tc_ld32(t_run + c0, w);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __float_as_uint(__uint_as_float(v[q]) + __uint_as_float(w[q]));
          } else {
            tc_wait_ld();
          }
          if (!last) {
            tc_st32(t_run + c0, v);
            continue;
          }
          const int n0 = tn * NS_BN + c0;
          if (row_ok && n0 < g.N) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int n = n0 + 4 * q;
              if (n < g.N) {  // N is a multiple of 4: a float4 is inside the row or outside it
                float4 o = make_float4(g.alpha * __uint_as_float(v[4 * q]), g.alpha * __uint_as_float(v[4 * q + 1]),
                                       g.alpha * __uint_as_float(v[4 * q + 2]), g.alpha * __uint_as_float(v[4 * q + 3]));
                if (drow) {
                  const float4 d = ld4(drow + n);
                  o.x = fmaf(g.beta, d.x, o.x); o.y = fmaf(g.beta, d.y, o.y); o.z = fmaf(g.beta, d.z, o.z); o.w = fmaf(g.beta, d.w, o.w);
                }
                st4(crow + n, o);
              }
            }
          }
        }
        if (!last) tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) ns_arrive(&sm.chunk_free);
      }
    }
  } else if (warp == NS_EPI_WARPS) {
    // ------------------------------------------------------------------ the issuing thread (one elected lane)
    if (elect_one()) {
      constexpr uint32_t IDESC = tc_idesc(NS_BN);
      long long kb_count = 0, cc = 0;
      bool dead = false;
      for (long long tile = blockIdx.x; tile < n_tiles && !dead && !sm.abort; tile += gridDim.x) {
        for (int kb = 0; kb < n_kb; ++kb, ++kb_count) {
          const int in_chunk = kb % NS_KCHUNK_BLOCKS;
          if (in_chunk == 0) {  // a new chunk overwrites the accumulator: the epilogue must be done with the previous one
            if (cc > 0 && !ns_wait(&sm.chunk_free, (uint32_t)((cc - 1) & 1), &sm.abort)) { dead = true; break; }
            tc_fence_after();
          }
          const int s = (int)(kb_count & 1);
          if (!ns_wait(&sm.full[s], (uint32_t)((kb_count >> 1) & 1), &sm.abort)) { dead = true; break; }
          tc_fence_after();
          const uint64_t ah = ns_desc(smem_addr(sm.st[s].a_hi)), al = ns_desc(smem_addr(sm.st[s].a_lo));
          const uint64_t bh = ns_desc(smem_addr(sm.st[s].b_hi)), bl = ns_desc(smem_addr(sm.st[s].b_lo));
          // one K step of 8 floats = 32 bytes further along the 128-byte row: the start address moves, the swizzle
          // is applied by the hardware to the address it computes
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) tc_mma_ss(tmem, al + 2 * ks, bh + 2 * ks, IDESC, (in_chunk > 0 || ks > 0) ? 1u : 0u);  // lo x hi
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) tc_mma_ss(tmem, ah + 2 * ks, bl + 2 * ks, IDESC, 1u);                                   // hi x lo
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) tc_mma_ss(tmem, ah + 2 * ks, bh + 2 * ks, IDESC, 1u);                                   // hi x hi
          tc_commit(&sm.empty[s]);
          if (in_chunk == NS_KCHUNK_BLOCKS - 1 || kb == n_kb - 1) { tc_commit(&sm.chunk_ready); ++cc; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ loaders: group 0 fills stage 0, group 1 stage 1
    const int lw = warp - NS_EPI_WARPS - 1, grp = lw >> 3, wg8 = lw & 7;
    NsStage& st = sm.st[grp];
    const int r4 = lane >> 3, c8 = lane & 7;  // a warp instruction covers 4 rows x 8 pieces of 16 bytes (whole 128-byte rows)
    long long kb_count = 0;
    bool dead = false;
    for (long long tile = blockIdx.x; tile < n_tiles && !dead && !sm.abort; tile += gridDim.x) {
      const int b = (int)(tile / tiles_per_batch), r = (int)(tile % tiles_per_batch);
      int tm, tn;
      ns_tile_coords(r, tiles_m, tiles_n, g.symmetric, tm, tn);
      const float* Ab = g.A + (long long)b * g.sA;
      const float* Bb = g.B + (long long)b * g.sB;
      for (int kb = 0; kb < n_kb; ++kb, ++kb_count) {
        if ((int)(kb_count & 1) != grp) continue;
        const int k = kb * NS_BK + 4 * c8;
        float4 v[12];
#pragma unroll
        for (int i = 0; i < 12; ++i) {
          const int u = wg8 + 8 * i;            // unit of 4 rows: 32 units for A, then 64 for B
          const bool isA = u < 32;
          const int row = (isA ? u : u - 32) * 4 + r4;
          const int grow = (isA ? tm * NS_BM : tn * NS_BN) + row;
          const bool ok = grow < (isA ? g.M : g.N) && k < g.K;   // K is a multiple of 4: a piece is inside or outside
          const float* src = (isA ? Ab + (long long)grow * g.lda : Bb + (long long)grow * g.ldb) + k;
          v[i] = ok ? ldg4(src) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const long long use = kb_count >> 1;  // how many times this stage has been filled before
        if (use > 0 && !ns_wait(&sm.empty[grp], (uint32_t)((use - 1) & 1), &sm.abort)) { dead = true; break; }
#pragma unroll
        for (int i = 0; i < 12; ++i) {
          const int u = wg8 + 8 * i;
          const bool isA = u < 32;
          const int row = (isA ? u : u - 32) * 4 + r4;
          const int off = ns_swz(row, c8) / 4;
          // high part = x rounded to the nearest TF32 value, low part = the exact remainder (the tensor core drops
          // its last bits): what is lost is at most 2^-23 of |x| and has no preferred sign; masking the low bits of x
          // off instead would lose up to 2^-22 and always downwards
          const float4 x = v[i];
          const float4 hi = make_float4(tf32_rn(x.x), tf32_rn(x.y), tf32_rn(x.z), tf32_rn(x.w));
          const float4 lo = make_float4(x.x - hi.x, x.y - hi.y, x.z - hi.z, x.w - hi.w);
          st4((isA ? st.a_hi : st.b_hi) + off, hi);
          st4((isA ? st.a_lo : st.b_lo) + off, lo);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) ns_arrive(&sm.full[grp]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sm.abort && status) atomicOr(status, 4);
  if (warp == NS_EPI_WARPS) tc_dealloc(tmem, 512);
}

// Batched 32 x 32-tile transposes through shared memory.
//   mode 0: dst[b][j][i] = src[b][i][j] for an [R][C] matrix (the x^T that the third product of a round reads);
//   mode 1: in place on a square [R][R] matrix: the part below the diagonal becomes the mirror image of the part above
//           it (completes the symmetric products; the diagonal tiles are mirrored inside the tile).
__global__ void __launch_bounds__(256) k_transpose32(const float* __restrict__ src, float* __restrict__ dst, int R, int C,
                                                     int lds, int ldd, long long ss, long long sd, int mode) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, ti = blockIdx.y, tj = blockIdx.x;
  if (mode == 1 && tj < ti) return;  // source tiles: on and above the diagonal
  const float* s = src + (long long)b * ss;
  float* d = dst + (long long)b * sd;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int i = ti * 32 + ty + 8 * q, j = tj * 32 + tx;
    if (i < R && j < C) tile[ty + 8 * q][tx] = s[(long long)i * lds + j];
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int j = tj * 32 + ty + 8 * q, i = ti * 32 + tx;   // destination element (j, i)
    if (i < R && j < C && (mode == 0 || j > i)) d[(long long)j * ldd + i] = tile[tx][ty + 8 * q];
  }
}
