/* hz_b200.h — C ABI of libhz_b200.so (CUDA sm_100a).
 *
 * Every entry point takes plain device pointers, a shape struct and a CUDA
 * stream (passed as void* so that this header needs no CUDA include), enqueues
 * work on that stream and returns an int status. Nothing here synchronises the
 * host with the device, throws, aborts or traps. All tensors are contiguous
 * row-major float32 unless stated; all buffers are owned by the caller.
 *
 * Reference citations are paths inside the HamiltonZero source tree.
 */
#ifndef HZ_B200_H_
#define HZ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define HZ_OK                 0
#define HZ_ERR_NULL_POINTER   1   /* a required pointer is NULL                  */
#define HZ_ERR_BAD_SHAPE      2   /* non-positive or inconsistent extent         */
#define HZ_ERR_UNSUPPORTED    3   /* extent outside what the kernels implement   */
#define HZ_ERR_MISALIGNED     4   /* pointer not aligned as required             */
#define HZ_ERR_CUDA           5   /* a CUDA runtime call failed; see hz_last_cuda_error */
#define HZ_ERR_NO_DEVICE      6   /* no usable sm_100 device                     */
#define HZ_ERR_WORKSPACE      7   /* caller-provided workspace is too small      */
#define HZ_ERR_STATIC_SCRATCH  8   /* problem exceeds the built-in scratch of hz_logpsi_static */
#define HZ_ERR_TIMEOUT        9   /* a bounded device-side wait ran out (hz_workspace_status)  */
#define HZ_ERR_WRONG_DEVICE  10   /* a buffer lives on another device than the current one     */

/* Human-readable text for a status code (static storage). */
const char* hz_status_string(int status);
/* cudaError_t value of the last failing runtime call made by this library on
 * the calling thread (0 if none). */
int hz_last_cuda_error(void);
/* Library version: major*10000 + minor*100 + patch. */
int hz_version(void);

/* Device-side waits (TMA completion, tensor-core commits) are bounded: a wait that runs out
 * (about two seconds) records a code in the first word of the call's workspace, the CTA frees
 * what it holds and returns, and the call's outputs are overwritten with NaN, so that a timeout
 * can never pass as a result. Nothing traps or faults. hz_workspace_status waits for `stream`
 * and returns HZ_OK or HZ_ERR_TIMEOUT for the last hz_logpsi / hz_local_energy /
 * hz_logpsi_vjp / hz_mcmc_sweep call that ran with `workspace`. The word is cleared at the
 * start of every such call. No counterpart in the reference (XLA reports device errors through
 * its own runtime). */
int hz_workspace_status(const void* workspace, void* stream);
/* Self-test of that path: enqueues one tiny kernel whose only wait can never be satisfied and
 * whose limit is about a millisecond; the wait runs out, the kernel records the code in the first
 * word of `workspace` (at least 256 bytes, 256-byte aligned) and returns. Afterwards
 * hz_workspace_status(workspace, stream) answers HZ_ERR_TIMEOUT; the next operator call that uses
 * the workspace clears the word. Nothing traps, faults or spins without bound. No counterpart in
 * the reference. */
int hz_selftest_wait_timeout(void* workspace, long long workspace_bytes, void* stream);

/* ---- large-N context path: rectangular attention and the 2-FWL ring panel ----
 * hz_mha_rect_fwd replaces noncausal_bias_mha (src/hamiltonzero/evaluation/pallas_mha.py:100-161)
 * as pallas_rectangular_edge_attention drives it
 * (src/hamiltonzero/evaluation/sequence_parallel.py:59-95): out = softmax_k(q k^T D^-1/2 + bias) v
 * over ALL keys, forward only, fp32. q [B, Lq, H, D] (unscaled: the D^-1/2 is applied inside),
 * k, v [B, Lk, H, D], bias [B, Lq, Lk, H], key_mask [B, Lk] bytes (0 = masked: that key's bias
 * is replaced by -1e30 as the caller does; null = no mask), out [B, Lq, H, D]. Any Lq, Lk >= 1;
 * H a multiple of 4 up to 16; D in {8, 16, 32, 64}; otherwise HZ_ERR_UNSUPPORTED.
 * workspace: hz_mha_rect_workspace_bytes(...) bytes of device scratch for the partial sums when
 * the keys are split over several CTAs (few query rows, many keys); with a null or smaller
 * workspace the keys are not split (same result, less parallelism). */
long long hz_mha_rect_workspace_bytes(int B, int Lq, int Lk, int H, int D);
int hz_mha_rect_fwd(int B, int Lq, int Lk, int H, int D, const float* q, const float* k,
                    const float* v, const float* bias, const uint8_t* key_mask, float* out,
                    void* workspace, long long workspace_bytes, void* stream);

/* One ring step of ring_learned_fwl2_columns_local
 * (src/hamiltonzero/evaluation/sequence_parallel.py:112-173):
 * out[i, j, c] (+)= sum_k a[i, k0 + k, c] * b_panel[k, j, c], with a [rows, a_cols, channels],
 * b_panel [panel, cols, channels], out [rows, cols, channels]; accumulate = 0 overwrites out. */
int hz_fwl2_panel(const float* a, const float* b_panel, float* out, int rows, int a_cols, int k0,
                  int panel, int cols, int channels, int accumulate, void* stream);

/* ---- per-stage device timing of the walker pipeline ----------------------
 * No counterpart in the reference, whose only timing is host wall-clock around
 * block_until_ready (src/hamiltonzero/modes/train.py:635-644). When enabled, each
 * stage launch of hz_logpsi / hz_local_energy is bracketed by CUDA events on the
 * caller's stream; hz_stage_timing_read waits for them and returns, per stage,
 * the accumulated milliseconds, algorithmic fp32 FLOPs and launch count
 * (arrays of at least hz_stage_count() entries; reset != 0 clears the totals). */
int hz_stage_count(void);
const char* hz_stage_name(int stage);
int hz_stage_timing_enable(int on);
int hz_stage_timing_read(double* ms, double* flops, long long* launches, int n, int reset);

/* ==== B1: masked multi-head softmax attention with additive edge bias ======
 *
 * Layouts (reference: src/hamiltonzero/model/_pallas_attn/mhsea_tuned.py:95-101,
 * 201-203): q,k,v,out,tangents,gradients [B,N,H,D]; e,et,de [B,N,H,N];
 * mask [B,N] one byte per token (non-zero = real token); lse [B,N,H].
 * q is the query already multiplied by D^-1/2, as the reference's dispatcher
 * passes it (src/hamiltonzero/model/pallas_attention.py:62).
 *
 * Supported extents: 1 <= N <= 256, D in {8,16,32,64}, any B,H >= 1.
 * Pointers to [B,N,H,D] and [B,N,H,N] tensors must be 16-byte aligned.
 *
 * mask_mode selects the masking convention:
 *   HZ_MASK_SQUARE  the Pallas kernels' convention: masked q/k/v rows are
 *                   zeroed before the dot products, masked (i,j) pairs score
 *                   -10000, masked query rows of the outputs are zero
 *                   (mhsea.py:13-31, utils.py:52-53, mhsea_tuned.py:91).
 *   HZ_MASK_KEYS    the einsum twin's convention: -1e9 is added to the scores
 *                   of masked keys and nothing else is masked
 *                   (pallas_attention.py:22-37).
 */
#define HZ_MASK_SQUARE 0
#define HZ_MASK_KEYS   1
/* Arithmetic of the contractions. The generic kernels (any N <= 256, D in {8,16,32,64}) always
 * use a three-term TF32 split, accurate to fp32 rounding. The whole-sequence kernels (N = 64,
 * D = 32, square mask) take, when no flag is given, a two-term BF16 split - three BF16 products
 * per fp32 product, fp32 accumulation, the range of fp32: every output stays within 1e-4 of its
 * scale (about 1e-5 for operands of order one), and the three passes run at the HBM rate. The
 * flags below, OR-ed into mask_mode, select another arithmetic there.
 *
 * HZ_ATTN_TF32: single-pass TF32 contractions, the arithmetic of the reference's Triton
 * kernels (tl.dot on fp32 operands; relative error of a score about 1e-3). */
#define HZ_ATTN_TF32   0x100
/* HZ_ATTN_TF32X3: the three-term TF32 split (fp32-faithful, about 1e-6 of scale) at half of the
 * tensor rate of the default. */
#define HZ_ATTN_TF32X3 0x1000
/* Optional flag, OR-ed into mask_mode, forward only: run the tcgen05 / TMEM / TMA forward kernel
 * where it applies (N = 64, D = 32, H even, square mask); it computes on the three-term TF32
 * split. At present slower than the default kernel (see the kernel's header), so it is a
 * permission, not the default. */
#define HZ_ATTN_TCGEN05 0x200
/* HZ_ATTN_BF16X3: names the default arithmetic explicitly (two-term BF16 split: each product
 * exact to about 3 * 2^-16 of its magnitude). HZ_ATTN_TF32 and HZ_ATTN_TF32X3 win if set as well. */
#define HZ_ATTN_BF16X3 0x400
/* Optional flag, OR-ed into mask_mode: the same split with FP16 heads and tails (11 significant
 * bits each). A product is exact to about 3 * 2^-22 of its magnitude, i.e. results sit as close to
 * the fp32 ones as with the default split (about 1e-6 of scale), at the speed of HZ_ATTN_BF16X3.
 * The caller guarantees that q, k, v, their tangents and the cotangent stay inside the FP16
 * range (|x| < 65504; a value beyond it contracts as infinity). HZ_ATTN_TF32 and HZ_ATTN_BF16X3
 * win if set as well. */
#define HZ_ATTN_FP16X3 0x800

typedef struct hz_attn_shape {
  int32_t B;          /* batch (any vmapped axes folded in, mhsea_tuned.py:121-163) */
  int32_t N;          /* tokens                                                      */
  int32_t H;          /* kernel heads                                                */
  int32_t D;          /* head dimension                                              */
  int32_t mask_mode;  /* HZ_MASK_SQUARE or HZ_MASK_KEYS [| HZ_ATTN_* flags]          */
} hz_attn_shape;

/* Primal: out, lse = MHSEA(q,k,e,v,mask).
 * Replaces mhsea_forward + mhsea_kernel
 * (src/hamiltonzero/model/_pallas_attn/custom_gradients.py:24-75, mhsea.py:13-31)
 * and the row zeroing of _outer_impl (mhsea_tuned.py:76-92), i.e. the lowering
 * of primitives mhsea_tuned_ad / mhsea_full_ad.
 * e and mask may be NULL (zero bias / all tokens real). */
int hz_mhsea_fwd(const hz_attn_shape* shape,
                 const float* q, const float* k, const float* e, const float* v,
                 const uint8_t* mask, float* out, float* lse, void* stream);

/* Linear tangent given the saved out, lse.
 * Replaces mhsea_tangent_pallas (mhsea_tuned_jvp.py:20-91,104-222) and
 * mhsea_jvp_pallas (mhsea_full_ad_jvp.py:19-109), i.e. the lowering of
 * primitives mhsea_tuned_ad_lin / mhsea_full_ad_lin (mhsea_tuned.py:179-198).
 * e, et and mask may be NULL. Masked query rows of the tangent are zero. */
int hz_mhsea_jvp(const hz_attn_shape* shape,
                 const float* q, const float* k, const float* e, const float* v,
                 const uint8_t* mask, const float* out, const float* lse,
                 const float* qt, const float* kt, const float* et, const float* vt,
                 float* tangent, void* stream);

/* Transpose of the tangent primitive: dq (w.r.t. the pre-scaled q), dk, de, dv.
 * Replaces mhsea_backward = mhsea_q_vjp_kernel + mhsea_kv_vjp_kernel
 * (custom_gradients.py:78-347), reached from _inner_transpose
 * (mhsea_tuned.py:206-221). e, mask and de may be NULL (de NULL: not written). */
int hz_mhsea_bwd(const hz_attn_shape* shape,
                 const float* q, const float* k, const float* e, const float* v,
                 const uint8_t* mask, const float* lse, const float* out,
                 const float* dout,
                 float* dq, float* dk, float* de, float* dv, void* stream);

/* ==== B2: walker-batch operators ===========================================
 *
 * The compiled binary-merge-tree wavefunction as plain device arrays: the fields of
 * SharedKernel and CompiledTree (src/hamiltonzero/compiled/types.py:38-45,131-140;
 * produced by src/hamiltonzero/compiled/trunk.py:26-35 and compiled/tree.py:96-303).
 * Per-level arrays are concatenated, first merge level (N/2 nodes) first.
 * Supported: n_sites a power of two <= 256, d_r = 32, d_m a multiple of 32,
 * r_leaf, r_merge, r_ro multiples of 4.
 */
typedef struct hz_wavefunction {
  int32_t n_sites;          /* N (routed, padded width)                               */
  int32_t d_o;              /* width of q_to_odd                                      */
  int32_t d_m;              /* carrier width (merge_dim)                              */
  int32_t d_r;              /* group width of merge_T; G = d_m / d_r                  */
  int32_t r_leaf, r_merge, r_ro;
  float merge_eps;          /* SharedKernel.merge_eps                                 */
  const float* q_weight;    /* [4, d_o]        kernel.q_to_odd.weight                 */
  const float* leaf_V;      /* [d_o, r_leaf]   kernel.leaf_factors[0].V               */
  const float* leaf_U;      /* [r_leaf, d_m]   kernel.leaf_factors[0].U               */
  const float* leaf_h;      /* [N, r_leaf]     tree.leaf_h[0]                         */
  const float* merge_T;     /* [G, d_r, d_r, d_r] kernel.merge_T                      */
  const float* merge_V;     /* [d_m, r_merge]  kernel.merge_factors[0].V              */
  const float* merge_U;     /* [r_merge, d_m]  kernel.merge_factors[0].U              */
  const float* merge_h;     /* sum_l [N>>(l+1), r_merge]  tree.merge_h, concatenated  */
  const uint8_t* opcodes;   /* sum_l [N>>(l+1)] tree.opcodes: 0 MERGE 1 CARRY_LEFT
                               2 CARRY_RIGHT 3 EMPTY (compiled/types.py:15-19)        */
  const float* readout_V;   /* [d_m, r_ro]     kernel.readout_factors[0].V            */
  const float* readout_U;   /* [r_ro, 2]       kernel.readout_factors[0].U            */
  const float* readout_h;   /* [r_ro]          tree.readout_h[0]                      */
} hz_wavefunction;

/* The routed energy frame (EnergyFrame, compiled/types.py:113-118, built by
 * src/hamiltonzero/energy/frame.py:122-141). The per-level blocks w_levels are
 * diagonal blocks of J_eff and are read from it directly. */
typedef struct hz_energy_frame {
  const float* J_eff;            /* [3N, 3N] custom_lap_J_eff (symmetric)              */
  const float* one_body_field;   /* [N, 3]   one_body_fields[0]                        */
  float radial_const;            /* custom_lap_radial_const                            */
} hz_energy_frame;

/* Bytes of caller-provided scratch needed to process `walkers_per_chunk` walkers
 * at a time (with_jets: 1 for hz_local_energy, 2 for hz_logpsi_grad, 0 for hz_logpsi); -1 on bad
 * arguments. Calls accept any workspace at least as large as the value for one
 * walker and split the batch into chunks that fit; results do not depend on the
 * chunk size (the role of chunk_size / lax.map batch_size in
 * src/hamiltonzero/energy/kernel.py:164-193). The workspace must be 256-byte aligned. */
long long hz_walker_workspace_bytes(const hz_wavefunction* wf, int with_jets,
                                    long long walkers_per_chunk);

/* log|psi| and phase of B routed walkers q [B, N, 4].
 * Replaces execute_wavefunction / CompiledWaveFunction.__call__
 * (src/hamiltonzero/compiled/execute.py:79-118, compiled/types.py:146-153). */
int hz_logpsi(const hz_wavefunction* wf, const float* q, long long B,
              float* log_abs, float* phase,
              void* workspace, long long workspace_bytes, void* stream);

/* log|psi|, phase and their chart gradient grad [B][3N][2] (d log|psi| / dz, d phase / dz in the
 * right-SU(2) chart at z = 0) of B routed walkers: one forward pass that carries the value and the
 * Jacobian rows only (no Laplacian, no energy frame). This is the derivative that the sampler
 * caches projected on the frame e_1..e_3 (src/hamiltonzero/mcmc/langevin.py:25-40,
 * src/hamiltonzero/mcmc/runtime.py:66-72: value_and_grad of 2 log|psi|) and that local_spin
 * takes by jacrev (src/hamiltonzero/observables.py:15-28): spin = -i/2 (grad_re + i grad_im). */
int hz_logpsi_grad(const hz_wavefunction* wf, const float* q, long long B,
                   float* log_abs, float* phase, float* grad,
                   void* workspace, long long workspace_bytes, void* stream);

/* Forward-Laplacian local energy of B routed walkers q [B, N, 4].
 * energies [4][B][2]: (re, im) of total, exchange, casimir, field.
 * log_abs, phase [B]: the wavefunction value, a by-product.
 * grad (nullable) [B][3N][2]: d(log|psi|)/dz and d(phase)/dz in the right-SU(2)
 * chart at z = 0, from which the spin estimator is -i/2 (grad_re + i grad_im).
 * Replaces vmc_energy_custom_lap_compiled (src/hamiltonzero/energy/compiled.py:17-31)
 * = _run_custom_lap_batch + _custom_lap_single_from_frame (energy/kernel.py:80-193)
 * + custom_forward_laplacian_with_jac (energy/custom_lap.py:1458-1482), and the
 * Jacobian that local_spin takes by jacrev (src/hamiltonzero/observables.py:15-59). */
int hz_local_energy(const hz_wavefunction* wf, const hz_energy_frame* frame,
                    const float* q, long long B, float* energies,
                    float* log_abs, float* phase, float* grad,
                    void* workspace, long long workspace_bytes, void* stream);

/* ---- reverse pass: parameter and walker gradients of (log|psi|, phase) ----------------------
 * Replaces the backward pass that JAX derives from CompiledFinetuneWaveFunction.call_tagged
 * (src/hamiltonzero/compiled/model.py:179-310) for the loss tangent of
 * src/hamiltonzero/optim/production.py:168-228:
 *     grads = sum_w ( cot_log_abs[w] * d log|psi_w| / d theta + cot_phase[w] * d phase_w / d theta )
 * for every parameter array theta of hz_wavefunction, and, when dq is not NULL,
 *     dq[w, site, :] = the same combination differentiated with respect to q[w, site, :]
 * (the ambient gradient that the sampler caches as grad_log_p, src/hamiltonzero/mcmc/runtime.py:66-72).
 * The arrays of hz_wavefunction_grads have the shapes of the arrays of hz_wavefunction with the
 * same name and are overwritten. log_abs and phase (nullable) receive the forward values. Gated
 * nodes (opcode other than MERGE) and padded leaves contribute nothing to the factor and tensor
 * gradients, which is the structural mask of the reference's tags. */
typedef struct hz_wavefunction_grads {
  float* q_weight;
  float* leaf_V;
  float* leaf_U;
  float* leaf_h;
  float* merge_T;
  float* merge_V;
  float* merge_U;
  float* merge_h;
  float* readout_V;
  float* readout_U;
  float* readout_h;
} hz_wavefunction_grads;

/* Optional KFAC factor statistics of the same backward pass (factors may be NULL, and so may
 * every pointer in it): for each dense tag of call_tagged the sum over walkers - and, for the
 * factors shared by all merge levels, over levels and nodes - of x x^T ("_in", x the layer's
 * input under the tag's structural mask) and of dy dy^T ("_out", dy the cotangent of the layer's
 * output), i.e. the sums that StructuralRepeatedDenseKroneckerFactored divides by its batch
 * sizes (src/hamiltonzero/optim/blocks.py:1122-1204); for each scale tag the sum over walkers
 * of the squared per-walker gradient of the scale ("_diag", blocks.py:1288-1415). All arrays are
 * overwritten. For the quadrilinear tag compiled.merge.T the sums behind the two-Kronecker
 * marginals of its curvature block (src/hamiltonzero/optim/spin_blocks.py:140-171,443-560) over
 * the balanced axis split (i, j | k, l) of T [G, d_r, d_r, d_r], MERGE nodes only:
 *   merge_T_left  [(i,j),(I,J)] = sum keep (a_i . a_I)(b_i . b_I) dy[i,j] dy[I,J]
 *   merge_T_right [(k,l),(K,L)] = sum keep sum_i |dy_i|^2 a[i,k] a[i,K] b[i,l] b[i,L]
 *   merge_T_stats = (sum keep sum_i |dy_i|^2 |a_i|^2 |b_i|^2, sum keep)
 * with dy the cotangent of the merge output and a, b the two children's carriers; the division
 * by the batch size, the trace normalisation and the moving averages stay with the optimiser.
 * Requesting either marginal costs about d_r^4 multiply-adds per (walker, node, group). */
typedef struct hz_kfac_factors {
  const uint8_t* leaf_mask;  /* [N] 1 = real leaf (leaf tags' structural mask); NULL = all real */
  float* q_in;               /* [4, 4]            compiled.q_to_odd                            */
  float* q_out;              /* [d_o, d_o]                                                     */
  float* leaf_V_in;          /* [d_o, d_o]        compiled.leaf.V                              */
  float* leaf_V_out;         /* [r_leaf, r_leaf]                                               */
  float* leaf_U_in;          /* [r_leaf, r_leaf]  compiled.leaf.U                              */
  float* leaf_U_out;         /* [d_m, d_m]                                                     */
  float* leaf_h_diag;        /* [N, r_leaf]       compiled.leaf.h                              */
  float* merge_V_in;         /* [d_m, d_m]        compiled.merge.V (MERGE rows)                */
  float* merge_V_out;        /* [r_merge, r_merge]                                             */
  float* merge_U_in;         /* [r_merge, r_merge] compiled.merge.U                            */
  float* merge_U_out;        /* [d_m, d_m]                                                     */
  float* merge_h_diag;       /* [(N-1) r_merge]   compiled.merge.h, level-major like merge_h   */
  float* readout_V_in;       /* [d_m, d_m]        compiled.readout.V                           */
  float* readout_V_out;      /* [r_ro, r_ro]                                                   */
  float* readout_U_in;       /* [r_ro, r_ro]      compiled.readout.U                           */
  float* readout_U_out;      /* [2, 2]                                                         */
  float* readout_h_diag;     /* [r_ro]            compiled.readout.h                           */
  float* merge_T_left;       /* [d_m, d_m]        compiled.merge.T, axes (i, j)                 */
  float* merge_T_right;      /* [d_r^2, d_r^2]    compiled.merge.T, axes (k, l)                 */
  float* merge_T_stats;      /* [2]               trace mass, number of merged (walker, node)   */
} hz_kfac_factors;

/* Bytes of workspace for hz_logpsi_vjp with `walkers_per_chunk` walkers per pass (about
 * 2.4 MB per walker at 64 sites with the default sizes, 0.4 MB more with factors); with_factors:
 * 0 none, 1 the dense and scale tags, 2 also the marginals of the quadrilinear tag (up to
 * 128 MB more); -1 for unsupported extents. */
long long hz_vjp_workspace_bytes(const hz_wavefunction* wf, long long walkers_per_chunk,
                                 int with_factors);

int hz_logpsi_vjp(const hz_wavefunction* wf, const float* q, long long B,
                  const float* cot_log_abs, const float* cot_phase,
                  const hz_wavefunction_grads* grads, const hz_kfac_factors* factors, float* dq,
                  float* log_abs, float* phase,
                  void* workspace, long long workspace_bytes, void* stream);

/* ---- replica-exchange MALA sweep on SU(2)^N ------------------------------------------------
 * State of B walkers x R replicas (REState, src/hamiltonzero/mcmc/replica_exchange.py:21-36),
 * structure of arrays, all device pointers. `drift` replaces the reference's cached
 * grad_log_p [R,N,4]: it is that gradient projected on the frame e_1..e_3
 * (src/hamiltonzero/mcmc/langevin.py:25-40), the only form in which the reference uses it.
 * The scalar counters n_local and n_haar of the reference advance by n_steps and 1 per sweep
 * and are kept by the caller, as is `step` (+ n_steps). */
typedef struct hz_mcmc_state {
  int32_t n_walkers, n_replicas, n_sites;
  int32_t step;              /* swap parity counter at entry                              */
  uint64_t seed;             /* Philox key                                                */
  uint64_t offset;           /* sweep counter: distinct offsets give independent draws    */
  float* q;                  /* [B, R, N, 4]                                              */
  float* log_p;              /* [B, R]    2 log|psi|                                      */
  float* drift;              /* [B, R, N, 3]                                              */
  const float* beta;         /* [R]  inverse temperatures, cold chain last                */
  const float* sigma;        /* [R]  proposal widths                                      */
  const int32_t* mask;       /* [N]  real sites                                           */
  const int32_t* m;          /* [R]  sites refreshed by the Haar move                     */
  float* n_local_accept;     /* [B, R]                                                    */
  float* n_swap_accept;      /* [B, R-1]                                                  */
  int32_t* n_swap;           /* [B, R-1]                                                  */
  float* n_haar_accept;      /* [B, R]                                                    */
} hz_mcmc_state;

/* Optional replacement of the internal random draws (any pointer may be NULL), used to check
 * single moves against a host restatement on identical numbers. */
typedef struct hz_mcmc_noise {
  const float* haar_scores;  /* [B, R, N]    U(0,1)                                       */
  const float* haar_raw;     /* [B, R, N, 4] N(0,1)                                       */
  const float* haar_logu;    /* [B, R]       log U(0,1)                                   */
  const float* local_noise;  /* [n_steps, B, R, N, 3] N(0,1)                              */
  const float* local_logu;   /* [n_steps, B, R]       log U(0,1)                          */
  const float* swap_logu;    /* [n_steps, B, R-1]     log U(0,1)                          */
} hz_mcmc_noise;

/* Scratch for hz_mcmc_sweep when the value-and-gradient passes run replicas_per_chunk
 * (walker, replica) pairs at a time; -1 on bad arguments. */
long long hz_mcmc_workspace_bytes(const hz_wavefunction* wf, int n_walkers, int n_replicas,
                                  long long replicas_per_chunk);

/* One sampler call: refresh of the cached (log p, drift), one global Haar move, then n_steps
 * x (one MALA move per replica + deterministic even-odd neighbour swaps).
 * Replaces run_batched -> run_re_langevin_cached (src/hamiltonzero/mcmc/runtime.py:88-129,
 * src/hamiltonzero/mcmc/replica_exchange.py:286-303) with langevin_step_one_cached
 * (langevin.py:84-135), _swap_move and _global_haar_step (replica_exchange.py:112-198).
 * Each value-and-gradient of log p is one forward-jet pass of the executor.
 * log_alpha_out (nullable) [n_steps, B, R] receives the MALA log acceptance ratios.
 * Random numbers are Philox4x32-10(seed, offset), not JAX's threefry: agreement with the
 * reference's sampler is distributional. */
int hz_mcmc_sweep(const hz_wavefunction* wf, hz_mcmc_state* state, int n_steps,
                  const hz_mcmc_noise* noise, float* log_alpha_out,
                  void* workspace, long long workspace_bytes, void* stream);

/* hz_logpsi for callers that cannot give the library memory and must not let it allocate.
 * This entry point has no counterpart in the reference. It exists for hosts such as a
 * plugin inside a runtime whose memory pool already owns the GPU (where a cudaMalloc made
 * by the plugin may fail, and blocks the whole device while it runs), or a binding that
 * receives input and output buffers only and has no scratch allocator to ask.
 *
 * Same arguments and results as hz_logpsi minus the workspace. The scratch is a fixed array
 * of hz_static_scratch_bytes() bytes (32 MiB) inside the library, held by every GPU that
 * loads the library until the process exits. The batch is cut into chunks that fit, so any
 * B is accepted; a wavefunction whose scratch for ONE walker exceeds the array is refused
 * with HZ_ERR_STATIC_SCRATCH (every supported n_sites fits at the default model sizes; a
 * carrier width of 8192 at 256 sites, for example, does not).
 * The call makes no cudaMalloc / cudaFree and calls no allocating routine; it returns
 * HZ_ERR_UNSUPPORTED while hz_stage_timing_enable(1) is in effect, because the timer
 * creates CUDA events.
 *
 * Every call uses the array of the device that is current when it is made: q, log_abs, phase,
 * the wavefunction's arrays and the stream must belong to that device (q, log_abs and phase are
 * checked: HZ_ERR_WRONG_DEVICE). The first call on each device looks up the array's device
 * address (cudaGetSymbolAddress, with that device current) and caches it; make that first call
 * before starting any stream capture on the device.
 * All calls on one device share the array. Nothing in it needs clearing between calls:
 * every scratch element is written before it is read within a call, so stale contents of
 * the previous call are harmless. Two calls that overlap on the same GPU (different
 * streams or host threads) race on the array and corrupt each other: serialise them. */
long long hz_static_scratch_bytes(void);
int hz_logpsi_static(const hz_wavefunction* wf, const float* q, long long B,
                     float* log_abs, float* phase, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HZ_B200_H_ */
