/*
 * cgnet_b200 -- C ABI of the B200 (sm_100a) Clebsch-Gordan layer library, libcgnet_b200.so.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns an int status (CGB200_OK == 0).
 * Device pointers are ordinary CUDA device addresses owned by the caller; nothing here allocates or frees a caller
 * buffer.  `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  No call synchronises the
 * device; work is ordered on `stream` only.  After a non-zero status, cgb200_last_error() (thread-local) says why.
 *
 * Data layout (the reference project's, zlin7/CGNet; file:line below are paths inside that project):
 *   activation   float[B][N][2]            N = sum_l tau_l (2l+1); fragment l starts at cum[l] = sum_{l'<l} tau_l'(2l'+1);
 *                                          inside it element (t, m) sits at t(2l+1) + (m+l); last axis (re, im)
 *                                          (CGNet/cudaCG/cudaCG_sparse.cu:17, CGNet/CGutils.py:190-197)
 *   triples      int32 codes (l(L+1)+l1)(L+1)+l2 with l2 <= l1, grouped by l, inside l ordered by l1
 *                                          (CGNet/CGutils.py:122-140)
 *   mid channel  of triple k in degree l:  t_offsets[k] + t1*tau_l2 + t2            (CGNet/CG_layers.py:253-262)
 *   CG table     float, per triple a (2l+1) x (2l2+1) band, entry [m+l][m2+l2] = <l1 m-m2; l2 m2 | l m>, zero when
 *                |m-m2| > l1                                                          (CGNet/cudaCG/cudaCG_sparse.cu:68-92)
 *   weights      float[sum_l tau_out[l] t_FF[l]][2]; degree l is a row-major (tau_out[l], t_FF[l]) complex matrix
 *                                          (CGNet/cudaCG/cudaCG_FNWMM.cu:18, CGNet/CG_layers.py:98)
 *   stds         float[sum_l t_FF[l]]      one moving standard deviation per mid channel (CGNet/CG_layers.py:116-117)
 */
#ifndef CGNET_B200_H_
#define CGNET_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CGB200_OK               0
#define CGB200_ERR_ARGUMENT     1   /* null pointer, negative size, misaligned buffer, inconsistent plan            */
#define CGB200_ERR_UNSUPPORTED  2   /* shape outside what the kernels handle (see cgb200_last_error)               */
#define CGB200_ERR_CUDA         3   /* a CUDA runtime call failed; the message carries cudaGetErrorString          */
#define CGB200_ERR_WORKSPACE    4   /* workspace too small                                                          */

/* fragment-norm flags, same bit meaning as the reference's `bn_flags` (CGNet/CG_layers.py:22-33) */
#define CGB200_FN_PRESENT       0x1 /* stds is valid: divide every mid channel by max(eps, stds[k])                */
#define CGB200_FN_UPDATE        0x2 /* training: first fold this batch's statistics into stds, in place            */
#define CGB200_FN_KEEP_MID      0x4 /* cgb200_layer_bwd only: the workspace is the one the matching cgb200_layer_fwd call
                                       (same plan, same batch, CGB200_FN_UPDATE set) used, untouched since, and at least
                                       cgb200_layer_workspace_bytes large: where cgb200_layer_keeps_mid says so, that forward
                                       left the tiles of the mid activation in it and the weight gradient reads them
                                       instead of generating them again.  Ignored where the forward keeps nothing.   */

/* plan flags */
#define CGB200_PLAN_DEPTHWISE   0x1 /* channel-wise product (t1 == t2 only; needs tau_l1 == tau_l2).  Not in the
                                       reference (its 'mst' mode keeps the full tau_l1 x tau_l2 product)           */
#define CGB200_PLAN_TILE(t)     (((t) & 0xF) << 8)  /* force the channel-tile edge (1..6) instead of the plan's choice   */

typedef struct cgb200_plan cgb200_plan;

const char* cgb200_last_error(void);
int cgb200_version(void);

/* Largest lmax accepted.  Replaces `sparse_maxL` (CGNet/cudaCG/cudaCG_all.cpp:124-126). */
int cgb200_max_lmax(void);

/*
 * Build the CG band table for a triple list on the device.
 * Replaces `sparse_precomputeCG` (CGNet/cudaCG/cudaCG_all.cpp:112-121 -> cudaCG_sparse.cu:304-319).
 *   cg_dev      device float[cg_len], fully overwritten (entries outside the band become 0)
 *   llls_host   HOST int32[n_llls] triple codes;  the offsets follow from them: off[k+1] = off[k] + (2l+1)(2l2+1)
 */
int cgb200_cg_table_build(float* cg_dev, int64_t cg_len, int lmax, const int32_t* llls_host, int n_llls, void* stream);
/* Length the table needs for a triple list (CGNet/CGutils.py:154-158). */
int64_t cgb200_cg_table_length(int lmax, const int32_t* llls_host, int n_llls);

/*
 * A plan holds everything that depends only on (lmax, tau_in, tau_out, triple list): the index tables the
 * reference keeps as seven int32 tensors on its module (CGNet/CG_layers.py:244-250, :104-108), the CG table
 * (CGNet/CG_layers.py:134-141) and the work lists of the kernels.  Host arrays are copied.  tau_out may be NULL
 * for a product-only plan.  The plan belongs to the CUDA device that is current when it is created.
 */
int  cgb200_plan_create(cgb200_plan** out, int lmax, const int32_t* tau_in, const int32_t* tau_out,
                        const int32_t* llls_host, int n_llls, int flags);
void cgb200_plan_destroy(cgb200_plan* plan);

/* Sizes derived by the plan, in complex elements per sample unless stated. */
#define CGB200_Q_N_F        0   /* input activation length                                    */
#define CGB200_Q_N_FF       1   /* CG-product (mid) activation length                         */
#define CGB200_Q_N_O        2   /* output activation length (0 without tau_out)               */
#define CGB200_Q_W_LEN      3   /* complex weights                                            */
#define CGB200_Q_SUM_TFF    4   /* mid channels = length of stds                              */
#define CGB200_Q_CG_LEN     5   /* floats in the CG table                                     */
#define CGB200_Q_N_TRIPLES  6
#define CGB200_Q_TILE       7   /* channel-tile edge chosen for the register-tiled kernels    */
int cgb200_plan_query(const cgb200_plan* plan, int what, int64_t* value);
/*
 * Device-side status of the plan's kernels (no reference counterpart).  The tensor-core kernels wait on hardware
 * barriers with an iteration limit; a wait that runs out makes the kernel give up: it sets this word, fills the part
 * of the output it owns with NaN (so a training loss shows the failure without a device synchronisation), releases
 * its tensor memory and returns.  The call synchronises the device, returns the word in *status (0 = fine) and clears it.
 */
int cgb200_plan_status(const cgb200_plan* plan, int32_t* status);
/*
 * Kernel selection of a plan (no reference counterpart: the reference has one kernel per step).  Every option starts
 * at CGB200_AUTO, the library's measured default for the plan's shape; 0 / 1 force a variant off / on where the plan has
 * its tables, otherwise the call returns CGB200_ERR_UNSUPPORTED.  Options are per plan, not per process, and take
 * effect from the next call; do not change them while a call on the same plan is being enqueued from another thread.
 */
#define CGB200_AUTO                 (-1)
#define CGB200_OPT_TC_FWD           0   /* forward on tcgen05 tensor cores (tile edge 2 or 4, full product)            */
#define CGB200_OPT_TC_GRAD_W        1   /* weight gradient on tensor cores (tile edge 4 or 5)                            */
#define CGB200_OPT_TC_GRAD_F        2   /* first phase of the input gradient on tensor cores (tile edge 4)               */
#define CGB200_OPT_TC_STAGES        3   /* upper limit of the tensor-core kernels' generator groups = pipeline stages (>= 2) */
#define CGB200_OPT_FWD_SLAB         4   /* CUDA-core forward: persistent blocks with the slab in shared memory           */
#define CGB200_OPT_GRAD_F_SPLIT     5   /* input gradient: rows of phase 2 split into two channel groups                 */
#define CGB200_OPT_STATS_SPLIT      6   /* statistics: two blocks per cell                                               */
#define CGB200_OPT_BWD_SERIAL       7   /* backward: weight and input gradient on one stream instead of forked           */
#define CGB200_OPT_WAIT_POLLS       8   /* iteration limit of every bounded device-side wait (default 4000000)           */
#define CGB200_OPT_TEST_IDLE_MMA    9   /* test hook: the tensor-core kernels' MMA warp issues nothing, so every wait on
                                           it runs out; exercises the give-up path (status word, NaN output) without a
                                           fault, a trap or an endless loop                                              */
#define CGB200_OPT_TC_STAGED        10  /* tensor-core forward, off by default: 1 = a staging warp bulk-copies each cell's CG
                                           band rows, operand rows and packed weights into a shared-memory ring ahead of the
                                           generators, 2 = band rows and weights only                                       */
#define CGB200_OPT_TC_ABUF          11  /* staged tensor-core forward: upper limit of the A-tile buffers (>= 2)                */
#define CGB200_OPT_TC_FWD_SPLIT     12  /* tensor-core forward: splitting level 0..6 of the contraction (the degree with the
                                           most cells in 2^level parts, partial outputs added in part order); default: by
                                           the batch size, so that the longest block stays a fraction of an SM's share      */
#define CGB200_OPT_GRAD_MID_GEMM    13  /* input gradient: the mid activation's gradient by a tensor-core GEMM into the
                                           workspace, read back by the input-gradient kernel, instead of rebuilt tile by
                                           tile on the CUDA cores (tile edge 4, full product); 2 / 3: on, with the kernel
                                           that reads the tiles forced to / kept from running two blocks per SM             */
#define CGB200_OPT_FWD_KEEP_MID      14  /* forward with a statistics update on the tensor-core path: the statistics kernel
                                           keeps the tiles of the mid activation it generates in the workspace and the
                                           forward kernel reads them back instead of generating them again               */
#define CGB200_OPT_SHORT_GROUP       15  /* CUDA-core weight gradient and input gradient: the idle lanes of a last sample
                                           group that is at most half full share its work (0: off)                       */
#define CGB200_OPT_COUNT            16
int cgb200_plan_set_option(cgb200_plan* plan, int option, int value);
int cgb200_plan_get_option(const cgb200_plan* plan, int option, int* value);

/* Per-degree mid-channel counts t_FF[0..lmax] (CGNet/CG_layers.py:253-262), for cross-checking the host's own. */
int cgb200_plan_t_ff(const cgb200_plan* plan, int32_t* t_ff_host);
/* Device address of the plan's CG table (float[CGB200_Q_CG_LEN]); valid until the plan is destroyed. */
const float* cgb200_plan_cg_table(const cgb200_plan* plan);

/*
 * CG product  F -> FF.   Replaces `sparse_forward` (CGNet/cudaCG/cudaCG_all.cpp:39-71 -> cudaCG_sparse.cu:96-184).
 *   F   device float[B][N_F][2]     FF  device float[B][N_FF][2], every element written
 */
int cgb200_cg_product_fwd(const cgb200_plan* plan, const float* F, float* FF, int64_t B, void* stream);

/*
 * Gradient of the CG product with respect to its input.
 * Replaces `sparse_backward` (CGNet/cudaCG/cudaCG_all.cpp:73-108 -> cudaCG_sparse.cu:186-298).
 *   gFF device float[B][N_FF][2]    gF  device float[B][N_F][2], every element written (no pre-zeroing needed)
 */
int cgb200_cg_product_bwd(const cgb200_plan* plan, const float* F, const float* gFF, float* gF, int64_t B, void* stream);

/*
 * Fragment norm + channel mixing  FF -> O.
 * Replaces `FN_WMM_forward` (CGNet/cudaCG/cudaCG_all.cpp:137-165 -> cudaCG_FNWMM.cu:29-123,215-245).
 *   flags & CGB200_FN_UPDATE: stds[k] <- stds[k]*cnt/(cnt+1) + sigma_k/(cnt+1) first, sigma_k the standard deviation
 *   of |FF[b,k,m]| over (b, m) computed in double; then O_l = W_l diag(1/max(eps, stds)) FF_l.
 *   stds may be NULL when CGB200_FN_PRESENT is clear.
 */
int cgb200_fn_wmm_fwd(const cgb200_plan* plan, const float* FF, const float* W, float* stds, float cnt, float eps,
                      int flags, float* O, int64_t B, void* stream);

/*
 * Gradients of the mixing.
 * Replaces `FN_WMM_backward` (CGNet/cudaCG/cudaCG_all.cpp:172-205 -> cudaCG_FNWMM.cu:126-211,250-282).
 *   gW  device float[W_LEN][2], fully written, summed over the batch in a fixed order (the reference uses atomicAdd)
 *   gFF device float[B][N_FF][2], fully written.  The statistics carry no gradient, as in the reference.
 */
int cgb200_fn_wmm_bwd(const cgb200_plan* plan, const float* gO, const float* FF, const float* W, const float* stds,
                      float eps, int flags, float* gFF, float* gW, int64_t B, void* stream);

/*
 * The whole layer in one pass, F -> O, without ever writing FF to memory.
 * Replaces the sequence `sparse_forward` + `FN_WMM_forward` issued by CGBN_cuda.forward (CGNet/CG_layers.py:313-318).
 * Same meaning of stds / cnt / eps / flags as cgb200_fn_wmm_fwd.
 *   workspace  device scratch of at least cgb200_layer_workspace_bytes(plan, B) bytes, 256-byte aligned, contents
 *              undefined on entry and exit.
 */
int cgb200_layer_fwd(const cgb200_plan* plan, const float* F, const float* W, float* stds, float cnt, float eps,
                     int flags, float* O, int64_t B, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Inference with weights that do not change between calls: the tensor-core forward multiplies by the weights in a packed
 * form (scaled by 1/max(eps, stds), real form, TF32 high / low parts, the MMA's operand order) that cgb200_layer_fwd
 * rebuilds on every call (4-14 % of a wide layer's forward).  Pack them once into a caller-owned buffer and call
 * cgb200_layer_fwd_packed: same result as cgb200_layer_fwd with the flags given here and without CGB200_FN_UPDATE, bit for
 * bit.  cgb200_layer_packed_weights_bytes is 0 for plans whose forward does not run on the tensor cores.  Pack again
 * after W, stds, eps or a plan option changes.
 */
int64_t cgb200_layer_packed_weights_bytes(const cgb200_plan* plan);
int cgb200_layer_pack_weights(const cgb200_plan* plan, const float* W, const float* stds, float eps, int flags,
                              void* packed, int64_t packed_bytes, void* stream);
int cgb200_layer_fwd_packed(const cgb200_plan* plan, const float* F, const void* packed, float* O, int64_t B,
                            void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Gradients of the whole layer, (F, W, stds, gO) -> (gF, gW), regenerating FF on the fly.
 * Replaces `FN_WMM_backward` + `sparse_backward` issued by autograd (CGNet/CG_layers.py:54-72, 194-203).
 * `stds` must be the values the forward used (i.e. after its update).  gF may be NULL when the gradient with respect
 * to the input is not wanted (the first layer of a network): that part of the work is then skipped.
 */
int cgb200_layer_bwd(const cgb200_plan* plan, const float* F, const float* W, const float* stds, float eps, int flags,
                     const float* gO, float* gF, float* gW, int64_t B, void* workspace, int64_t workspace_bytes,
                     void* stream);

/* Scratch bytes the two fused calls need for a batch of B samples (the larger of the two).  From 12 output channels on
   (tile edge 4, full product) the backward keeps the gradient of the mid activation in the workspace between its two
   kernels: 8 bytes per sample and element of the tile-padded mid activation, i.e. gigabytes for the wide layers (2.1 GB
   at lmax 14 with 16 channels and 64 samples; above 16 GB the library goes back to rebuilding it tile by tile;
   CGB200_OPT_GRAD_MID_GEMM 0 does so always). */
int64_t cgb200_layer_workspace_bytes(const cgb200_plan* plan, int64_t B);
/* 1 if a cgb200_layer_fwd call with CGB200_FN_UPDATE for B samples leaves the mid activation's tiles at the start of its
   workspace (tensor-core path, tile edge 4, see CGB200_OPT_FWD_KEEP_MID), so that cgb200_layer_bwd may be given the same
   workspace with CGB200_FN_KEEP_MID; 0 otherwise. */
int cgb200_layer_keeps_mid(const cgb200_plan* plan, int64_t B);
/* Scratch bytes cgb200_layer_fwd alone needs (input slab, norm factors, row counters, packed tensor-core weights);
   never more than cgb200_layer_workspace_bytes.  Both depend on the plan's options at the time of the call. */
int64_t cgb200_layer_fwd_workspace_bytes(const cgb200_plan* plan, int64_t B);
/* The same for a call with these flags: a forward without CGB200_FN_UPDATE keeps no tiles and needs no room for them
   (gigabytes less for the wide layers).  cgb200_layer_fwd accepts a workspace of that smaller size for any call: a forward
   with an update then generates its tiles twice instead of keeping them (and the backward must not be told
   CGB200_FN_KEEP_MID). */
int64_t cgb200_layer_fwd_workspace_bytes_for(const cgb200_plan* plan, int64_t B, int flags);

/*
 * cgb200_layer_fwd for callers that cannot allocate device memory (no counterpart in the reference, whose Python
 * layer always allocates through torch).  Same arguments and results, minus the workspace: the scratch is a fixed
 * array of CGB200_STATIC_SCRATCH_BYTES inside the library, resident on every GPU that loads it for the life of the
 * process.  Meant for hosts where an allocation is impossible or forbidden at call time: a plugin running inside
 * another runtime's callback, a process whose device memory belongs to a foreign arena, a service that bans
 * cudaMalloc after start-up because it stalls the device.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - Returns CGB200_ERR_WORKSPACE, with the needed and available byte counts in cgb200_last_error(), when
 *     cgb200_layer_fwd_workspace_bytes_for(plan, B, 0) exceeds the array (kept tiles are not used here).
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress with that device current);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps whatever the last call left in it.  The call itself
 *     rewrites everything it reads (nothing needs to be zeroed by the caller), but two calls whose kernels overlap on
 *     the GPU - different streams, or different threads - race on it: serialise them on one stream.
 */
#define CGB200_STATIC_SCRATCH_BYTES (8u << 20)
int cgb200_layer_fwd_static(const cgb200_plan* plan, const float* F, const float* W, float* stds, float cnt, float eps,
                            int flags, float* O, int64_t B, void* stream);

/*
 * Spherical-harmonic projection of sampled real functions, the step in front of the network:
 *     coefs[r][c] = scale * sum_p f[r][p] * basis[p][c]        (complex basis and result, real samples)
 * Replaces the contraction of `get_sph_coefs` (utils/s2_sph.py:79-86, basis = quadrature weight x conj(Y_lm) on the grid,
 * scale = 4 pi / P) and of `get_coef_C` (utils/geometries.py:125-144, basis = Y_lm at the sample points), which the
 * reference evaluates with numpy one function at a time; here all `rows` functions go through one tensor-core GEMM
 * (3xTF32, rounded partial sums).  The basis is packed once per (point set, lmax):
 *   basis         device float[n_points][n_cols][2]
 *   packed        device buffer of cgb200_sh_basis_bytes(n_points, n_cols) bytes, 256-byte aligned
 *   f             device float[rows][n_points]          coefs  device float[rows][n_cols][2], fully written
 *   workspace     cgb200_sh_workspace_bytes(rows, n_points) bytes, 256-byte aligned, contents undefined
 *   status_word   device int32, zero on entry; set to 1 if a bounded device-side wait ran out (coefs are then NaN)
 */
int64_t cgb200_sh_basis_bytes(int64_t n_points, int n_cols);
int64_t cgb200_sh_workspace_bytes(int64_t rows, int64_t n_points);
int cgb200_sh_basis_pack(const float* basis, int64_t n_points, int n_cols, float* packed, void* stream);
int cgb200_sh_project(const float* f, int64_t rows, int64_t n_points, int n_cols, const float* packed, float scale,
                      float* coefs, void* workspace, int64_t workspace_bytes, int32_t* status_word, void* stream);

/*
 * Mesh -> sphere projection by ray casting (the SHREC17 front end).  One ray per grid point g, from g towards the origin;
 * the first triangle it meets gives image[0][p] = distance from g to the hit (1 without a hit), image[1][p] = n . g and
 * image[2][p] = |n ^ g| (0 without a hit), n the triangle's unit normal from its winding, g normalised.
 * Replaces `render_model` (Shrec17/dataset.py:53-95), which takes the intersections from the trimesh package.
 *   vertices   device float[n_vertices][3]     faces  device int32[n_faces][3] (an index outside the vertices drops the face)
 *   sgrid      device float[n_points][3]       image  device float[3][n_points], fully written
 *   workspace  cgb200_raycast_workspace_bytes(n_faces) bytes, 256-byte aligned
 *   status_word  device int32, zero on entry; set to 1 if a bounded device-side wait ran out (those pixels are NaN)
 */
int64_t cgb200_raycast_workspace_bytes(int64_t n_faces);
int cgb200_raycast_sphere(const float* vertices, int64_t n_vertices, const int32_t* faces, int64_t n_faces, const float* sgrid,
                          int64_t n_points, float* image, void* workspace, int64_t workspace_bytes, int32_t* status_word,
                          void* stream);

/* Number of kernels this library launched in this process since the last reset (bench accounting). */
int64_t cgb200_launch_count(int reset);

/*
 * Optional per-kernel timing for benchmarks (no reference counterpart).  While enabled (process-wide), every
 * kernel launch is bracketed by CUDA events on its stream.  cgb200_timing_read waits for the recorded launches and
 * returns, per kernel id in [0, cgb200_kernel_count()), the summed device time in milliseconds and the number of
 * launches; `reset` non-zero forgets the recorded launches.  Do not enable it inside a CUDA-graph capture.
 */
int cgb200_kernel_count(void);
const char* cgb200_kernel_name(int kernel_id);
void cgb200_timing_enable(int on);
int cgb200_timing_read(double* ms_per_kernel, int64_t* launches_per_kernel, int reset);

#ifdef __cplusplus
}
#endif
#endif  /* CGNET_B200_H_ */
