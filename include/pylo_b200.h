/*
 * pylo_b200 - C ABI of the B200 (sm_100a) learned-optimizer step kernels.
 *
 * One shared library, plain C linkage, raw device pointers and sizes, a CUDA
 * stream passed as void*.  Every entry point returns an int:
 *   0            ok
 *   < 0          an argument was rejected on the host before anything was launched
 *   > 0          a cudaError_t reported by the launch
 * No entry point allocates, frees, synchronises or throws, unless its comment
 * says otherwise.  The caller owns all memory.  Descriptor, tile and item arrays
 * are DEVICE pointers; pylo_step_params and pylo_velo_rnn are HOST pointers whose
 * contents are copied into the launch.  Calls are re-entrant as long
 * as two calls in flight do not share workspace.
 *
 * The three pybind functions of the reference that this library replaces:
 *   cuda_lo.learned_optimizer_kernel      pylo/csrc/learned_optimizer.cu:303-404
 *   celo2_cuda_kernel.celo2_kernel        pylo/csrc/celo2_kernel.cu:284-357
 *   velo_cuda_kernel.velo_kernel_simple   pylo/csrc/velo_kernel.cu:370-462
 * together with the torch-op state update the reference's Python classes run
 * before calling them (pylo/optim/AdafacLO_cuda.py:322-373,
 * pylo/optim/CELO2_cuda.py:205-232, pylo/optim/velo_cuda.py:502-546).
 *
 * The work is described by two tables in DEVICE memory that the host builds
 * once per parameter set: an array of pylo_tensor_desc (one per parameter
 * tensor) and arrays of tiles that cut the tensors into units of work.  One
 * optimizer step is a fixed sequence of launches over those tables
 * (see pylo_b200_* below, in call order).
 */
#ifndef PYLO_B200_H
#define PYLO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PYLO_B200_ABI_VERSION 10

/* optimizer families (which feature set / network geometry a launch uses) */
#define PYLO_FAM_ADAFAC 0 /* AdafacLO_CUDA, ELO_CUDA: 28+11 features, 39-32-32-2 */
#define PYLO_FAM_CELO2 1  /* CELO2_CUDA, ELO_CELO2_CUDA: 30 features, 30-8-8-3, writes step_out */
#define PYLO_FAM_VELO 2   /* VeLO_CUDA: 30 features, 30-4-4-3, per-tensor weights */

/* how a tensor is traversed */
#define PYLO_MODE_FAST2D 0  /* contiguous [X,Y], Y % 4 == 0, 16-byte aligned: float4 path */
#define PYLO_MODE_GENERIC 1 /* any contiguous [O,X,M,Y,I] view, scalar loads */
#define PYLO_MODE_VEC1D 2   /* fewer than two dims: accumulators are full size ("vector_like") */

#define PYLO_STAT_STRIDE 40  /* floats per tile partial / per tensor sums: 30 feature slots + 8 VeLO statistics */
#define PYLO_TILE_ELEMS 16384 /* elements per element-wise tile */
#define PYLO_A_COLS 1024      /* columns per row/column-sum tile */
#define PYLO_WFOLD_STRIDE 2432 /* floats reserved per tensor for the folded network */
#define PYLO_MAX_PEERS 7       /* other GPUs of one box */

/*
 * One unit of element-wise work: a whole parameter tensor, or one matrix slice of a tensor
 * with more than two dims when the normalisers are taken per slice (CELO2 family,
 * CELO2_naive.py:328-329).  A slice points into its tensor's buffers (idx0, m_stride) and
 * shares its factor vectors.  The tensor is viewed as a contiguous 5-D array
 * [O, X, M, Y, I]; X and Y are its two factored axes in memory order and O, M,
 * I the products of the other axes.  "a" vectors drop the Y axis (length
 * O*X*M*I, indexed by x for a 2-D tensor), "b" vectors drop the X axis (length
 * O*M*Y*I, indexed by y).  r_is_a says whether the reference's row accumulator
 * (exp_avg_sq_r / fac_r / fac_vec_row, which drops axis dr) is the "a" one.
 */
typedef struct pylo_tensor_desc {
  const float* g; /* gradient [n] */
  float* p;       /* parameter [n] */
  float* m;       /* momentum [3][n] */
  float* v;       /* second moment [n] */
  float* fac_a;   /* factored accumulator state, [3][La] (VEC1D: the row one, [3][n]) */
  float* fac_b;   /* factored accumulator state, [3][Lb] (VEC1D: the column one or NULL) */
  float* f_a;     /* workspace [3][La]: rsqrt factor in "a" orientation */
  float* f_b;     /* workspace [3][Lb] */
  float* fx;      /* workspace [La][4]: f_a interleaved per index (FAST2D only) */
  float* sum_a;   /* workspace [La]: sum over Y of g'^2 + 1e-30 */
  float* sum_b;   /* workspace [Lb]: sum over X */
  float* part_a;  /* workspace [X][n_cb]  row-sum partials (FAST2D) */
  float* part_b;  /* workspace [n_strips][Y] column-sum partials (FAST2D) */
  float* h_a;     /* workspace [La][H] (ADAFAC) or [La][H][2] (CELO2, VELO): first-layer term of the "a" features (+ bias) */
  float* h_b;     /* workspace [H][Lb]: first-layer term of the "b" features */
  float* closed;  /* workspace [PYLO_STAT_STRIDE]: closed-form sums of squares of vector features */
  float* sums;    /* workspace [48]: per-tensor sums (30 feature slots, 8 VeLO statistics, their 8 low-order parts) */
  float* wfold;   /* workspace [PYLO_WFOLD_STRIDE]: network with normalisers folded in */
  float* tile_part; /* workspace [n_tiles][PYLO_STAT_STRIDE] */
  float* out;     /* CELO2: raw step output [n]; else NULL */
  const float* w; /* network weights for this tensor, family layout (see pylo_b200_prep_apply) */
  const float* lr_mult; /* VeLO: device scalar multiplying lr for this tensor, else NULL */
  float* p_peer[PYLO_MAX_PEERS]; /* the same parameter inside the other ranks' peer-mapped buffers (first n_peer
                                    entries valid): kernels that write p store the new value there as well, which
                                    replaces the all-gather of updated parameters.  n_peer < 0: p_peer[0] is a
                                    multicast address mapping the parameter in every rank's buffer, and the kernels
                                    issue one multimem store to it instead */
  int64_t n;        /* elements of this unit */
  int64_t m_stride; /* distance in floats between the three momentum planes (n for a whole tensor) */
  int64_t idx0;     /* offset of this unit's first element inside the [O,X,M,Y,I] view (0 for a whole tensor) */
  int64_t La, Lb;   /* lengths of the "a" and "b" vectors (0 for VEC1D) */
  int32_t O, X, M, Y, I;
  int32_t mode;
  int32_t r_is_a;
  int32_t rcm_pre, rcm_A, rcm_post; /* row_col_mean: the row accumulator viewed [pre][A][post], mean over A */
  int32_t rb, n_strips, n_cb;       /* FAST2D phase-A tiling: rows per strip, strips, column blocks */
  int32_t tile0, n_tiles;           /* this tensor's range in the element-wise tile list */
  int32_t vec_elementwise;          /* 1: this unit is a slice of a tensor (its normalisers cover the slice only),
                                       so the vector-only features are accumulated per element, not in closed form */
  float lr;                         /* learning rate of the tensor's group */
  float wd;                         /* weight decay (family meaning) */
  float step;                       /* AdafacLO/ELO: 0-based step for the time features */
  float clip_norm;                  /* >0: scale g by clip_norm / max(global norm, clip_norm) */
  float exp_mult, step_mult;
  int32_t n_peer;                   /* number of valid p_peer entries (0: single GPU, or parameters gathered by NCCL) */
  int32_t pad_;
} pylo_tensor_desc;

/* a unit of element-wise work: elements [start, start + PYLO_TILE_ELEMS) of tensor `tensor` */
typedef struct pylo_tile {
  int64_t start;
  int32_t tensor;
  int32_t pad_;
} pylo_tile;

/* a unit of row/column-sum work: rows [row0, row0+rb) x columns [col0, col0+PYLO_A_COLS) */
typedef struct pylo_atile {
  int32_t tensor;
  int32_t strip;
  int32_t cb;
  int32_t pad_;
} pylo_atile;

/* per-launch constants shared by all tensors */
typedef struct pylo_step_params {
  int32_t family;
  int32_t nan_to_num;     /* ELO: torch.nan_to_num on the (scaled) gradient */
  int32_t wd_mode;        /* 0 none in kernel; 1 AdafacLO (after update, on new p); 2 ELO (on old p); 3 VeLO (lr_eff) */
  float step_delta;       /* added to every desc.step: lets the host advance the step count without re-uploading the table */
  float w_m[3];           /* 1 - beta_m[k], computed in fp32 as the reference does */
  float w_v;              /* 1 - beta_rms */
  float w_f[3];           /* 1 - beta_fac[k] */
  float eps_v;            /* added to g^2 before the second-moment EMA (1e-30 AdafacLO/ELO, 0 otherwise) */
  float eps_feat;         /* inside rsqrt(v + eps): 1e-6 AdafacLO/ELO/VeLO, 1e-8 CELO2 */
  float eps_norm;         /* inside rsqrt(S/n + eps): 1e-5 AdafacLO/ELO/VeLO, 1e-9 CELO2 */
  float clip_val;         /* element-wise clamp of the gradient; +inf for none */
  int32_t no_tables;      /* prep_apply: 0 = make the per-row (desc.h_a) and per-column (desc.h_b) first-layer tables,
                             1 = neither, 2 = the per-row table only (what the tensor-core apply kernel reads) */
  const float* gnorm_sq;  /* device scalar: sum of squares of all gradients, or NULL */
} pylo_step_params;

int pylo_b200_abi_version(void);
int pylo_b200_sizeof_desc(void);
int pylo_b200_sizeof_params(void);

/* Workspace sizing, for hosts that fill pylo_tensor_desc themselves.  The reference needs no counterpart: its
 * only scratch is the second_moment[28|30] tensor its Python classes allocate per call
 * (AdafacLO_cuda.py:376-380, CELO2_cuda.py:287-291, velo_cuda.py:731-735).
 *
 * pylo_b200_workspace_layout fills, for one tensor of the given family, traversal mode and geometry, the size
 * in floats of every workspace sub-buffer that pylo_tensor_desc points at (0 where the mode does not use it),
 * and the phase-A tiling (rb, n_strips, n_cb) and the number of element-wise tiles that go into the descriptor.
 * A unit of element-wise work that is a slice of a tensor (vec_elementwise = 1) owns only the last three
 * sub-buffers (sums, wfold, tile_part), sized with n = the slice's elements, plus a zero-filled `closed`; the
 * others belong to its tensor.  Every sub-buffer must start on a 256-byte boundary and the whole workspace
 * must be zero before the first step.
 * pylo_b200_workspace_bytes adds the sizes up, each rounded up to 256 bytes: tensor_part != 0 counts f_a .. closed,
 * unit_part != 0 counts sums, wfold, tile_part.  Host-only; nothing is launched. */
typedef struct pylo_ws_layout {
  int64_t f_a, f_b, sum_a, sum_b, fx, part_a, part_b, h_a, h_b, closed; /* per tensor */
  int64_t sums, wfold, tile_part;                                         /* per unit of element-wise work */
  int32_t rb, n_strips, n_cb, n_tiles;
} pylo_ws_layout;
int pylo_b200_workspace_layout(int family, int mode, int64_t n, int64_t La, int64_t Lb, int32_t X, int32_t Y,
                               pylo_ws_layout* out);
int64_t pylo_b200_workspace_bytes(const pylo_ws_layout* layout, int tensor_part, int unit_part);

/* Sum of squares of every gradient (CELO2_cuda.py:180-188, ELO_cuda.py:150-158).
 * items: one per tensor with a gradient (all of them, AdamW-routed ones included);
 * tiles: element-wise tiles over the items; scratch: [n_tiles] floats; out: device scalar. */
typedef struct pylo_gvec {
  const float* g;
  int64_t n;
} pylo_gvec;
int pylo_b200_grad_sumsq(const pylo_gvec* items, const pylo_tile* tiles, int n_tiles,
                         float* scratch, float* out, void* stream);

/* The same sum of squares for callers that cannot provide scratch memory (no counterpart in the
 * reference: it never needs scratch because it reduces with atomics).
 *
 * Who needs it: a host that cannot allocate device memory for us - for example a binding from another
 * language that links nothing but this library, or an optimizer hook that is forbidden to call
 * cudaMalloc inside the step because cudaMalloc stalls the whole device.  This entry point calls no
 * cudaMalloc / cudaFree and no allocating library routine; the per-tile partial sums go to a fixed
 * array inside the library (PYLO_STATIC_SCRATCH_TILES floats = 256 KiB, resident on every GPU that
 * loads the library until the process ends).
 *
 * Limits and rules:
 *  - n_tiles <= PYLO_STATIC_SCRATCH_TILES (2^16 tiles = 2^30 gradient elements); more is refused with
 *    PYLO_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched.
 *  - The first call on each device looks up the array's device address (with that device current).
 *    Make that first call during set-up, before any stream capture begins.
 *  - All calls share the one array, and it keeps whatever the previous call left in it.  That is
 *    harmless here (each call overwrites every slot it later reads, so nothing needs zeroing), but two
 *    calls that overlap on the GPU - different streams, or different host threads - race on it and
 *    give wrong sums.  Serialise them.
 * items, tiles, out, stream: as for pylo_b200_grad_sumsq. */
#define PYLO_STATIC_SCRATCH_TILES 65536
#define PYLO_ERR_STATIC_SCRATCH_TOO_SMALL (-4)
int pylo_b200_grad_sumsq_static(const pylo_gvec* items, const pylo_tile* tiles, int n_tiles, float* out,
                                void* stream);

/* Phase A: row and column sums of g'^2 + 1e-30 (the reductions inside
 * grad_sqr.mean(dim=dr / dc), AdafacLO_cuda.py:333-340, CELO2_cuda.py:218-224, velo_cuda.py:531-541).
 * atiles cover the FAST2D tensors (strip x 1024-column block each; they leave per-strip column partials);
 * rtiles, one per (FAST2D tensor, 1024-column block), drive the second-level sum of those partials over the
 * strips; generic_ids lists the GENERIC tensors. */
int pylo_b200_rowcol_sums(const pylo_tensor_desc* descs, const pylo_atile* atiles, int n_atiles,
                          const pylo_atile* rtiles, int n_rtiles, const int32_t* generic_ids, int n_generic,
                          const pylo_step_params* prm, void* stream);

/* Phase A2, one CTA per tensor: EMA of the factored accumulators, row_col_mean,
 * row/column rsqrt factors (AdafacLO_cuda.py:342-345, CELO2_cuda.py:229-231, velo_cuda.py:716-729)
 * and the closed-form feature moments of the twelve vector-only features. */
int pylo_b200_factor_update(const pylo_tensor_desc* descs, int n_tensors, const pylo_step_params* prm,
                            void* stream);

/* Phase B: momentum / second-moment EMA in place and per-tile sums of squares of
 * every element-wise feature (AdafacLO_cuda.py:341,370-373; lo_kernel learned_optimizer.cu:100-190;
 * celo2_moment_kernel celo2_kernel.cu:130-199; velo_compute_moments_kernel velo_kernel.cu:170-256).
 * For VeLO it also accumulates the statistics of the state before the update that
 * lstm_features_for_tensor needs (velo_cuda.py:213-252). */
int pylo_b200_state_moments(const pylo_tensor_desc* descs, const pylo_tile* tiles, int n_tiles,
                            int reverse, const pylo_step_params* prm, void* stream);

/* Phase B2, one CTA per tensor: fixed-order reduction of the tile partials into desc.sums. */
int pylo_b200_finalize_moments(const pylo_tensor_desc* descs, int n_tensors, void* stream);

/* Phase P, gridDim (n_tensors, slices): fold the normalisers rsqrt(S_j/n + eps) and, for
 * AdafacLO/ELO, the time features tanh(t/tau - 1) (learned_optimizer.cu:27-32,245-248) into the
 * first layer, and tabulate the first-layer contribution of the vector-only features.
 * desc.w layouts: ADAFAC  w_in[32][39] b_in[32] w_h[32][32] b_h[32] w_out[2][32] b_out[2] (out-major);
 *                 CELO2   w_in[30][8]  b_in[8]  w_h[8][8]   b_h[8]  w_out[8][3]  b_out[3] (in-major);
 *                 VELO    w_in[4][30]  b_in[4]  w_h[4][4]   b_h[4]  w_out[3][4]  b_out[3] (out-major). */
int pylo_b200_prep_apply(const pylo_tensor_desc* descs, int n_tensors, const pylo_step_params* prm,
                         void* stream);

/* Phase C: rebuild the features, run the network, write the parameter (ADAFAC, VELO) or the raw
 * step (CELO2) (lo_kernel_apply learned_optimizer.cu:194-301, celo2_apply_kernel celo2_kernel.cu:204-282,
 * velo_apply_kernel velo_kernel.cu:260-368). */
int pylo_b200_apply(const pylo_tensor_desc* descs, const pylo_tile* tiles, int n_tiles, int reverse,
                    const pylo_step_params* prm, void* stream);

/* Phase C for the FAST2D tensors of the ADAFAC family (same arithmetic as pylo_b200_apply, organised for
 * the FMA-bound 39-32-32-2 network: a thread keeps one column, packed fp32x2 FMAs).  ctiles: one entry per
 * tile with strip = row-tile index, cb = column-tile index, pad_ = columns per CTA (32, 64, 128 or 256) | (n_sub << 16); a work item
 * covers n_sub sub-tiles of 32 rows in one column block.  With this kernel in use pylo_b200_apply gets only the non-FAST2D tiles.
 * With one of the FAST2D kernels in use pylo_b200_apply handles the GENERIC and VEC1D units only. */
int pylo_b200_apply_adafac_cols(const pylo_tensor_desc* descs, const pylo_atile* ctiles, int n_ctiles,
                                const pylo_step_params* prm, void* stream);

/* Phase C for the FAST2D tensors of the ADAFAC family on the tensor cores (no reference counterpart: the
 * reference evaluates the network with scalar FMAs, lo_kernel_apply learned_optimizer.cu:236-284).  Same inputs
 * and outputs as pylo_b200_apply_adafac_cols, except that of the two first-layer tables it reads only desc.h_a
 * (run pylo_b200_prep_apply with no_tables = 2 or 0).  The two hidden layers run as tcgen05 TF32 products with
 * every operand split into a high and a low TF32 part (hi x hi + hi x lo + lo x hi), which keeps a 32-term dot
 * product within ~3e-7 of the sum of its terms' magnitudes; non-finite features give NaN where the scalar path may
 * give an infinity.  ttiles: strip = row-strip index, cb = block of 128 columns, pad_ = rows per work item (one
 * warpgroup of a CTA takes a whole item).  status: device int; the kernel ORs 1 into it if a wait on the tensor
 * core ran out (the parameters it could not finish then keep their old values), and a launch that finds it
 * non-zero stores nothing; may be NULL. */
int pylo_b200_apply_adafac_tc(const pylo_tensor_desc* descs, const pylo_atile* ttiles, int n_ttiles,
                              const pylo_step_params* prm, int* status, void* stream);

/* Phase C for the FAST2D tensors of the CELO2 and VELO families (same arithmetic as pylo_b200_apply, done on
 * pairs of adjacent elements with packed fp32x2 instructions).  ctiles: strip = row-tile index, cb = column-tile
 * index, pad_ = threads per row (8 .. 256, a thread owns 4 columns); a tile has 16 * (256 / pad_) rows and
 * 4 * pad_ columns.  For these families pylo_b200_prep_apply stores desc.h_a as (v, v) pairs, [X][H][2], and
 * for every family desc.h_b transposed, [H][Y]. */
int pylo_b200_apply_packed(const pylo_tensor_desc* descs, const pylo_atile* ctiles, int n_ctiles,
                           const pylo_step_params* prm, void* stream);

/* Batched fp32-faithful matrix product on the tensor cores, for the Newton-Schulz orthogonalisation of the CELO2
 * family (orthogonalize_via_newton_schulz, CELO2_naive.py:59-73, called at CELO2_cuda.py:332-335; the reference runs
 * it as torch.matmul):
 *     C[b][m][n] = alpha * sum_k A[b][m][k] * B[b][n][k] + beta * D[b][m][n]        b < batch
 * A is [M][K] with row pitch lda, B is [N][K] with row pitch ldb (both with K contiguous), C and D are [M][N].
 * One round of the iteration is three calls: a = x x^T (A = B = x), b = c1 a + c2 a a (A = B = D = a, a being
 * symmetric) and x' = c0 x + b x (A = b, B = x^T, D = x).  Every operand element is split into a TF32 high and low
 * part inside the kernel and three tcgen05 products (lo x hi, hi x lo, hi x hi) are accumulated in fp32.
 * Requirements (else -1): K, N and all pitches and batch strides multiples of 4, all pointers 16-byte aligned,
 * D (may be NULL) different from C.  g is a HOST pointer.  status: device int, bit 2 is ORed in if a bounded wait
 * inside the kernel ran out (the output is then incomplete); may be NULL. */
typedef struct pylo_gemm_desc {
  const float* A;
  const float* B;
  float* C;
  const float* D;
  int64_t strideA, strideB, strideC, strideD; /* distance in floats between consecutive matrices of the batch */
  int32_t M, N, K, lda, ldb, ldc, ldd, batch;
  float alpha, beta;
  int32_t symmetric; /* != 0: M == N and the result is symmetric (x x^T, a a): only the tiles that touch the diagonal or
                        lie above it are computed; complete C with pylo_b200_transpose(mirror = 1) afterwards */
  int32_t pad_;
} pylo_gemm_desc;
int pylo_b200_gemm_tn_3xtf32(const pylo_gemm_desc* g, int* status, void* stream);

/* Batched transposes for the Newton-Schulz chain.  mirror == 0: dst[b][j][i] = src[b][i][j] for [rows][cols]
 * matrices (src != dst).  mirror != 0: in place on square matrices (src == dst): everything below the diagonal
 * becomes the mirror image of what is above it. */
int pylo_b200_transpose(const float* src, float* dst, int rows, int cols, int ld_src, int ld_dst, int64_t stride_src,
                        int64_t stride_dst, int batch, int mirror, void* stream);

/* CELO2 tail (CELO2_cuda.py:336-339): step * rsqrt(mean(step^2 over the last two axes) + 1e-9) * rmsmult,
 * then p -= lr * (step + wd * p).  Items are matrices (the last two axes of a tensor). */
typedef struct pylo_post_item {
  const float* step; /* [n] orthogonalised (or raw) step */
  float* p;          /* [n] */
  float* part;       /* workspace [n_tiles] */
  int64_t n;
  int32_t tile0, n_tiles;
  float lr, wd, rmsmult, pad_;
} pylo_post_item;
int pylo_b200_celo2_post_sums(const pylo_post_item* items, const pylo_tile* tiles, int n_tiles, void* stream);
int pylo_b200_celo2_post_apply(const pylo_post_item* items, const pylo_tile* tiles, int n_tiles, void* stream);

/* AdamW branch for 1-D / embedding tensors.
 * independent != 0: CELO2_cuda.py:234-253 (own exp_avg/exp_avg_sq, betas b1,b2, bias correction with step t);
 * independent == 0: ELO_CELO2_cuda.py:244-253 (updates shared mom[3]/rms with prm, steps from mom[0], rms). */
typedef struct pylo_adam_item {
  const float* g;
  float* p;
  float* m; /* independent: exp_avg [n]; shared: mom [3][n] */
  float* v; /* independent: exp_avg_sq [n]; shared: rms [n] */
  int64_t n;
  float lr, wd, bc1, bc2; /* lr = adam_lr_mult*lr; bc = 1 - beta^t */
  float clip_norm, pad_[3];
} pylo_adam_item;
int pylo_b200_adamw(const pylo_adam_item* items, const pylo_tile* tiles, int n_tiles, int independent,
                    float beta1, float one_minus_beta1, float beta2, float one_minus_beta2, float eps,
                    const pylo_step_params* prm, void* stream);

/* VeLO front end.  velo_tensor_features: desc.sums -> the [T][30] LSTM input rows, row T-1-t for
 * tensor t (velo_cuda.py:213-252,419-422); loss features and fraction features are passed in.
 * When the tensors are sharded over ranks, descs holds this rank's n_local tensors, layer_of[i] is the
 * position of local tensor i among all n_total tensors (NULL: identity), rank_onehot is [n_local][5]; the
 * caller zeroes x_in first and sums it over the ranks afterwards.
 * velo_rnn: mix layers, LSTM cell, control and step-size heads, bank mixing (VeLO_RNN.py:110-135,
 * VeLO_MLP.py:92-126).  Outputs: weights [T][160] (row per tensor, tensor order), lr_mult [T]. */
typedef struct pylo_velo_rnn {
  const float *mix2_w, *mix2_b, *fmix_w, *fmix_b; /* [H][30], [H] */
  const float *lstm_w, *lstm_b;                   /* [4H][2H], [4H] */
  const float *ctrl_w, *ctrl_b;                   /* [B][H], [B] */
  const float *step_w, *step_b;                   /* [H], [1] */
  const float* bank;                              /* [B][159] */
  float *h, *c;                                   /* [T][H] LSTM state, updated in place */
  float *x_in;                                    /* [T][30] */
  float *pooled;                                  /* workspace [H] */
  float *xmix;                                    /* workspace [T][H] */
  float *gates;                                   /* workspace [T][4H] */
  float *controls;                                /* workspace [T][B] */
  float *weights;                                 /* out [T][160] */
  float *lr_mult;                                 /* out [T] */
  int32_t T, H, B, pad_;
} pylo_velo_rnn;
int pylo_b200_velo_tensor_features(const pylo_tensor_desc* descs, int n_local, const int32_t* layer_of,
                                   int n_total, const float* rank_onehot, const float* fraction9,
                                   const float* loss9, float* x_in, void* stream);
int pylo_b200_velo_rnn(const pylo_velo_rnn* rnn, void* stream);
/* BufferLossAccumulators.update + features (velo_cuda.py:183-211) on device; state arrays are the
 * loss_buffer tensors means[10], iteration (int32), running_min[10], decays[10]; writes loss9[9]. */
int pylo_b200_velo_loss_features(float* means, int32_t* iteration, float* running_min, const float* decays,
                                 const float* loss, float* loss9, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PYLO_B200_H */
