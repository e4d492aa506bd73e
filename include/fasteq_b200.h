/*
 * fasteq_b200 -- C ABI of the B200 (sm_100a) kernels for the equivariant
 * message-passing hot path.  Plain pointers and sizes only; every pointer is a
 * DEVICE pointer unless its comment says "host".  All launches are asynchronous
 * on the stream that is passed (a cudaStream_t cast to void*; NULL = default
 * stream) of the CURRENT device.  Functions return a fasteq_status; no C++
 * exception crosses this boundary (same contract as the reference's
 * EqLinearBackendApi, fasteq/cuda/src/eqlinear/common/eqlinear_common.h:16-22).
 *
 * Two kinds of shared library export these symbols:
 *   - libfasteq_b200_core.so : graph utilities, spherical harmonics, SO3Linear.
 *   - one generated module per operator signature (fasteq_u1d_* / fasteq_stc_*):
 *     the Clebsch-Gordan path table is compiled into the kernel, so each
 *     signature is its own .so exporting the same symbol names.
 */
#ifndef FASTEQ_B200_H_
#define FASTEQ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FASTEQ_ABI_VERSION 1

typedef enum fasteq_status {
  FASTEQ_OK = 0,
  FASTEQ_UNSUPPORTED = 1,   /* shape / mode this build does not implement */
  FASTEQ_INVALID = 2,       /* bad argument (null pointer, negative size, misalignment) */
  FASTEQ_CUDA_ERROR = 3,    /* a CUDA runtime call failed; see fasteq_last_cuda_error() */
  FASTEQ_INTERNAL = 4,
  FASTEQ_DEVICE_FAULT = 5   /* a kernel reported a bounded-wait timeout or an out-of-range index */
} fasteq_status;

typedef enum fasteq_dtype { FASTEQ_F32 = 0, FASTEQ_F64 = 1 } fasteq_dtype;

typedef void* fasteq_stream_t;

/* ------------------------------------------------------------------------- *
 * Uniform1D (ChannelwiseTensorProduct) generated modules.
 *
 * Replaces the pybind `run(w, x, y, [src_idx], [dst_idx], V)` entry point of the
 * reference's JIT modules (fasteq/ops/auto_schedule/uniform1d_forward.py:78-92,
 * 172-245) and the backward `run(w, x, y, grad_out, [src], [dst], V)`
 * (test/nequip_allegro_test/generated_uniform1d_bwd_lars.cu:246-324).
 *
 *   out[r_out, v, u] += c_p * w[r_w, i_p, u] * x[r_x, j_p, u] * y[r_y, k_p, u or 0]
 *
 * Tensors are contiguous [rows, segments, u].  Differences from the reference
 * entry point, all on the caller's side of the boundary: outputs are allocated
 * by the caller; the receiver index arrives as CSR segment offsets over
 * receiver-sorted edges (seg_ptr, see fasteq_graph_build_csr) plus an optional
 * permutation for unsorted input, instead of a raw dst index.
 * ------------------------------------------------------------------------- */
typedef struct fasteq_u1d_desc {
  int32_t abi_version;
  int32_t dtype;            /* fasteq_dtype */
  int32_t u, w_segs, x_segs, y_segs, out_segs, num_paths;
  int32_t y_vec;            /* 1: y is [rows, y_segs, u]; 0: y is [rows, y_segs, 1] */
  int32_t w_shared;         /* 1: w has a single row */
  int32_t x_indexed, y_indexed, scattered;
  int32_t direction;        /* 0 forward module, 1 backward module */
  int32_t need_gw, need_gx, need_gy;   /* backward modules: which gradients are produced */
  int32_t ctas_per_sm;      /* resident CTAs per SM the kernel was built for (grid = SMs * ctas_per_sm) */
  int32_t threads, smem_bytes;
} fasteq_u1d_desc;

typedef struct fasteq_u1d_graph {
  int64_t n_edges;          /* rows of the per-edge operands */
  int64_t n_out_rows;       /* rows of out (scattered: receivers; else == n_edges) */
  int64_t x_rows, y_rows;   /* rows of x and y (bounds for the gather indices) */
  const int32_t* x_index;   /* [n_edges] row of x per edge, or NULL (row = edge) */
  const int32_t* y_index;   /* [n_edges] row of y per edge, or NULL */
  const int32_t* seg_ptr;   /* [n_out_rows+1] CSR offsets into the receiver-sorted edge order (scattered only) */
  const int32_t* perm;      /* [n_edges] edge id at each sorted position, or NULL when edges are already sorted */
  const int32_t* part_ptr;  /* [n_parts+1] first segment (scattered) or first edge (else) of each CTA, or NULL = even split */
  int32_t n_parts;
} fasteq_u1d_graph;

int fasteq_u1d_describe(fasteq_u1d_desc* out /* host */);

/* out is fully overwritten (rows without edges become zero); no zero-fill needed. */
int fasteq_u1d_forward(const fasteq_u1d_graph* g /* host */, const void* w, const void* x, const void* y,
                       void* out, fasteq_stream_t stream);

/* Forward without any allocation (forward modules only).  No counterpart in the reference, whose
 * entry points allocate their outputs and leave scatter to atomics.  For callers that cannot
 * allocate device memory when they need the operator -- a plug-in of a simulation engine that
 * owns a fixed device arena, or a loop where an allocation's implicit synchronisation is not
 * acceptable.  Takes the receiver index itself (non-decreasing,
 * [n_edges]) and derives the CSR offsets and the per-CTA partition into an array built into the
 * module (about 1 MB PER MODULE, i.e. per operator signature, reserved on every GPU that loads the
 * module, shared by all calls into it), then runs the same kernel as fasteq_u1d_forward.  Limits: n_out_rows <= 262144 (else FASTEQ_UNSUPPORTED and
 * fasteq_last_cuda_error() names the limit); scattered signatures with y not gathered; edges already
 * sorted by receiver.  Calls that overlap on the GPU race on the shared array -- serialise them; a
 * refused call launches nothing and cannot disturb a call in flight.  Receiver indices outside
 * [0, n_out_rows) are not reported: such edges belong to no row and are left out (as with
 * fasteq_graph_build_csr).  The first call on each device resolves the array's device address (safe
 * from several host threads at once); make it before any stream capture.  Calls no cudaMalloc /
 * cudaFree or other allocating routine. */
int fasteq_u1d_forward_noalloc(const int32_t* dst_sorted, const int32_t* x_index, int64_t n_edges,
                               int64_t n_out_rows, int64_t x_rows, const void* w, const void* x, const void* y,
                               void* out, fasteq_stream_t stream);

/* grad_w / grad_x / grad_y may be NULL when the module was built without that gradient.
 * Gradients that are accumulated through an index (grad_x, grad_y when gathered, grad_w when
 * shared, grad_y when u is tiled) are zero-filled by this call on `stream` before the kernel. */
int fasteq_u1d_backward(const fasteq_u1d_graph* g /* host */, const void* grad_out, const void* w, const void* x,
                        const void* y, void* grad_w, void* grad_x, void* grad_y, fasteq_stream_t stream);

/* Reads and clears the device-side status word of this module (synchronises the device).
 * 0 = no fault; otherwise the code of the first fault (1 wait timeout, 2 index out of range). */
int fasteq_u1d_device_status(int32_t* code /* host */);

/* ------------------------------------------------------------------------- *
 * Symmetric tensor contraction (STC Uniform1D) generated modules.
 *
 *   out[b, v, u] = sum_p c_p * prod_t x1[b, a_{p,t}, u] * x0[i0[b], d_p, u]
 *
 * x1 [batch, x1_segs, u], x0 [n_species, x0_segs, u], i0 int32 [batch], out [batch, out_segs, u].
 * Replaces the pybind `run(x1, x0_g, V)` / `run(grad_out, x1, x0_g, V)` of the reference's JIT
 * modules (fasteq/ops/stc_uniform1d_jit.py:857,1070); the species gather x0[i0] is done inside.
 * ------------------------------------------------------------------------- */
typedef struct fasteq_stc_desc {
  int32_t abi_version, dtype, u, x1_segs, x0_segs, out_segs, num_paths;
  int32_t direction;   /* 0 forward module, 1 backward module */
  int32_t need_gx0;    /* backward: also writes the per-node weight gradient */
} fasteq_stc_desc;

int fasteq_stc_describe(fasteq_stc_desc* out /* host */);
int fasteq_stc_forward(const void* x1, const void* x0, const int32_t* i0, int64_t batch, int64_t n_species, void* out,
                       fasteq_stream_t stream);
/* grad_x1 [batch, x1_segs, u] is fully overwritten.  grad_x0_per_node [batch, x0_segs, u] (modules
 * built with need_gx0; else pass NULL) holds each node's contribution; the caller sums rows of equal
 * species (the reference does the same with index_add_, stc_uniform1d_jit.py:883-886). */
int fasteq_stc_backward(const void* grad_out, const void* x1, const void* x0, const int32_t* i0, int64_t batch,
                        int64_t n_species, void* grad_x1, void* grad_x0_per_node, fasteq_stream_t stream);
/* Second order (modules built for direction 2; others return FASTEQ_UNSUPPORTED): with ggx1 [batch, x1_segs, u] and
 * ggx0_per_node [batch, x0_segs, u] the cotangents of grad_x1 and of the per-node grad_x0, writes the
 * gradients of <ggx1, grad_x1> + <ggx0, grad_x0> with respect to grad_out, x1 and (per node) x0.
 * Replaces the reference's double-backward launcher run(go, x1, x0, i0, ggx0, ggx1, V) -> (dgo, dx1, dx0)
 * (fasteq/ops/stc_uniform1d_jit.py:964-968). */
int fasteq_stc_double_backward(const void* grad_out, const void* x1, const void* x0, const int32_t* i0, const void* ggx1,
                               const void* ggx0_per_node, int64_t batch, int64_t n_species, void* d_grad_out, void* d_x1,
                               void* d_x0_per_node, fasteq_stream_t stream);
int fasteq_stc_device_status(int32_t* code /* host */);

/* ------------------------------------------------------------------------- *
 * Spherical harmonics generated modules (one per degree list / dtype / normalisation):
 * vec [n, 3] -> out [n, sum(2l+1)], and the gradient with respect to vec.  Replaces the
 * reference's Triton kernels behind fasteq/triton/spherical_harmonics.py:493-570.
 * ------------------------------------------------------------------------- */
int fasteq_sh_num_outputs(void);
int fasteq_sh_forward(const void* vec, int64_t n, void* out, fasteq_stream_t stream);
int fasteq_sh_backward(const void* vec, const void* grad_out, int64_t n, void* grad_vec, fasteq_stream_t stream);
/* Second order: with ggvec [n, 3] the cotangent of grad_vec, d_grad_out[i] = <dY_i/dvec, ggvec> and
 * d_vec = sum_i grad_out[i] (d2Y_i / dvec dvec) ggvec (the reference's double backward uses an analytic
 * Hessian-vector product for the same purpose, fasteq/triton/spherical_harmonics.py:368-383). */
int fasteq_sh_double_backward(const void* vec, const void* grad_out, const void* ggvec, int64_t n, void* d_grad_out, void* d_vec,
                              fasteq_stream_t stream);

/* ------------------------------------------------------------------------- *
 * Core library.
 * ------------------------------------------------------------------------- */
const char* fasteq_status_string(int status);
const char* fasteq_last_cuda_error(void);
int fasteq_core_abi_version(void);

/* sorted_flag[0] (device int32) <- 1 if dst is non-decreasing else 0. */
int fasteq_graph_check_sorted(const int32_t* dst, int64_t n_edges, int32_t* sorted_flag, fasteq_stream_t stream);

/* CSR offsets of a non-decreasing receiver index: seg_ptr[r] = first position with dst >= r,
 * seg_ptr[n_rows] = n_edges.  Receiver indices outside [0, n_rows) are not reported: edges with a negative
 * index fall before row 0 and edges with an index >= n_rows after the last row, so no segment contains them
 * and the operators silently leave them out (there is no status word for this; validate the index on the
 * caller's side if it may be wrong).  The reference scatters with atomicAdd on the raw dst index
 * (fasteq/ops/auto_schedule/uniform1d_forward.py:351-356) and has no counterpart. */
int fasteq_graph_build_csr(const int32_t* dst_sorted, int64_t n_edges, int64_t n_rows, int32_t* seg_ptr,
                           fasteq_stream_t stream);

/* Split segments into n_parts contiguous ranges of about equal WORK, the work of a segment being its edge
 * count plus one (a receiver without edges still costs a row store): part_ptr[p] = first segment s with
 * seg_ptr[s] + s >= p * (n_edges + n_rows) / n_parts, part_ptr[n_parts] = n_rows. */
int fasteq_graph_partition(const int32_t* seg_ptr, int64_t n_rows, int64_t n_edges, int32_t n_parts,
                           int32_t* part_ptr, fasteq_stream_t stream);

/* ------------------------------------------------------------------------- *
 * Periodic radius graph on the GPU (a neighbour of the hot path; the reference's callers bring edge
 * lists from ASE / matscipy and it has no counterpart).  Batches of orthorhombic periodic boxes;
 * every pair (sender j, receiver i, image) with |r_j + shift - r_i| < cutoff, both directions, no
 * self edge in the home image, ordered by (receiver, sender, shift_x, shift_y, shift_z).  The count
 * step also yields the CSR offsets (seg_ptr) that fasteq_u1d_graph wants.
 *
 *   fasteq_neighbors_work_bytes(&p, &bytes);                          host only
 *   fasteq_neighbors_count(&p, work, bytes, seg_ptr, max_deg, s);     seg_ptr[n_atoms] = number of edges
 *   ... read seg_ptr[n_atoms] (and max_deg <= 1024), allocate the edge arrays ...
 *   fasteq_neighbors_fill(&p, work, bytes, seg_ptr, src, dst, shift, s);
 *
 * Positions are FP64 and must lie inside [0, box); distances are formed as ((r_j + shift) - r_i) with
 * individually rounded FP64 operations, so the edge set equals a numpy evaluation of the same formula.
 * ------------------------------------------------------------------------- */
typedef struct fasteq_nl_problem {
  int64_t n_atoms;
  int32_t n_structs;
  double cutoff;
  const double* pos;            /* device [n_atoms, 3] */
  const int32_t* atom_struct;   /* device [n_atoms] structure id of each atom */
  const double* box;            /* HOST [n_structs, 3] box lengths */
} fasteq_nl_problem;
int fasteq_neighbors_work_bytes(const fasteq_nl_problem* p /* host */, int64_t* bytes /* host */);
int fasteq_neighbors_count(const fasteq_nl_problem* p /* host */, void* work, int64_t work_bytes, int32_t* seg_ptr /* [n_atoms+1] */,
                           int32_t* max_degree /* device, may be NULL */, fasteq_stream_t stream);
int fasteq_neighbors_fill(const fasteq_nl_problem* p /* host */, void* work, int64_t work_bytes, const int32_t* seg_ptr,
                          int32_t* edge_src, int32_t* edge_dst, double* edge_shift /* [n_edges, 3] */, fasteq_stream_t stream);

/* ------------------------------------------------------------------------- *
 * SO3Linear ("eqlinear", subscripts uv,iu,iv): per-irrep channel mix
 *
 *   out[b, out_row[q] + t, :] += coeff[q] * x[b, in_row[q] + t, :] @ W[q]      t < rows[q]
 *
 * x is [batch, in_rows, u], W is [num_paths, u, v], out is [batch, out_rows, v], all contiguous.
 * Replaces the forward_create / forward_run / dgrad_* entries of the reference's
 * EqLinearBackendApi (fasteq/cuda/src/eqlinear/common/eqlinear_backend_api.h:12-27; problem layout
 * eqlinear_common.h:30-62; path mapping (input_row, output_row, weight_path, rows) :32-37).
 * The small path tables are host arrays read during the call.  The plain calls prepare the weights on the
 * fly; fasteq_eqlinear_pack + the _packed calls below let a caller keep the prepared form instead.
 * ------------------------------------------------------------------------- */
typedef enum fasteq_eqlinear_precision {
  FASTEQ_EQLIN_TF32X3 = 0,   /* FP32 data, 3xTF32 split on tensor cores (error < 2e-5 rel. Frobenius) */
  FASTEQ_EQLIN_FP32 = 1,     /* FP32 data, FP32 FMA */
  FASTEQ_EQLIN_FP64 = 2      /* FP64 data: DMMA (even extents, 16-byte aligned operands) or FP64 FMA */
} fasteq_eqlinear_precision;

typedef struct fasteq_eqlinear_problem {
  int32_t precision;          /* fasteq_eqlinear_precision */
  int32_t u, v;               /* channels in / out */
  int32_t in_rows, out_rows;  /* I = rows of x per batch entry, J = rows of out per batch entry */
  int32_t num_paths;          /* <= 64 */
  int64_t batch;
  const int32_t* in_row;      /* host [num_paths] first row of x the path reads */
  const int32_t* out_row;     /* host [num_paths] first row of out the path writes */
  const int32_t* rows;        /* host [num_paths] 2l+1 */
  const double* coeff;        /* host [num_paths] */
} fasteq_eqlinear_problem;

/* out is fully overwritten (rows no path writes become zero). */
int fasteq_eqlinear_forward(const fasteq_eqlinear_problem* p /* host */, const void* w, const void* x, void* out,
                            fasteq_stream_t stream);
/* grad_x[b, in_row[q]+t, :] = sum over paths reading that row of coeff[q] * grad_out[b, out_row[q]+t, :] @ W[q]^T
 * (the reference exposes grad_x only, eqlinear_runtime.py:86-104). grad_x is fully overwritten. */
int fasteq_eqlinear_dgrad(const fasteq_eqlinear_problem* p /* host */, const void* w, const void* grad_out,
                          void* grad_x, fasteq_stream_t stream);
/* Weights prepared once for many calls of the tensor-core path (FASTEQ_EQLIN_TF32X3): pre-scaled, K-major,
 * split into their two TF32 parts; packed holds 2 * num_paths * u * v floats; dgrad != 0 prepares the
 * grad_x layout.  The packed forms depend on the paths and coefficients but not on batch.  The _packed
 * calls return FASTEQ_UNSUPPORTED for shapes the tensor-core kernel does not take (use the plain calls).
 * Plays the part of the reference's forward_create / dgrad_create plan objects
 * (fasteq/cuda/src/eqlinear/common/eqlinear_backend_api.h:12-27), owned by the caller. */
int fasteq_eqlinear_pack(const fasteq_eqlinear_problem* p /* host */, int32_t dgrad, const void* w, void* packed,
                         fasteq_stream_t stream);
int fasteq_eqlinear_forward_packed(const fasteq_eqlinear_problem* p /* host */, const void* packed, const void* x, void* out,
                                   fasteq_stream_t stream);
int fasteq_eqlinear_dgrad_packed(const fasteq_eqlinear_problem* p /* host */, const void* packed, const void* grad_out,
                                 void* grad_x, fasteq_stream_t stream);
/* grad_w[q] = coeff[q] * sum_b sum_{t < rows[q]} x[b, in_row[q]+t, :]^T grad_out[b, out_row[q]+t, :]   ([u, v] per path).
 * Needed to train the mixing weights.  The reference's public operator returns no weight gradient
 * (eqlinear_runtime.py:104); its FP32 back-end keeps a reduction kernel for one
 * (fasteq/cuda/src/eqlinear/backends/fp32/reduce_dw.cu:12).  FP32 (also for FASTEQ_EQLIN_TF32X3) or FP64
 * FMA arithmetic, two deterministic stages: per-chunk partial sums in a stream-ordered temporary, then
 * their reduction.  grad_w [num_paths, u, v] is fully overwritten. */
int fasteq_eqlinear_wgrad(const fasteq_eqlinear_problem* p /* host */, const void* x, const void* grad_out,
                          void* grad_w, fasteq_stream_t stream);

/* The same operator in the shape of the reference's backend interface: a table of function pointers per precision,
 * field for field the EqLinearBackendApi / EqLinearProblemC / EqLinearPathC / EqLinearPlanInfo of
 * fasteq/cuda/src/eqlinear/common/eqlinear_backend_api.h:12-27 and eqlinear_common.h:30-62 (abi_version 2), so that a
 * dispatcher written against it (dispatch/eqlinear_dispatch.cpp:215-312) can load this library as a backend.
 * i_dims / paths / cg are borrowed during create only.  A plan owns a device copy of the weights in the form its kernel
 * multiplies with (create calls cudaMalloc and enqueues the preparation on `stream`), is bound to the problem's batch
 * size B, and must be destroyed by the same table's destroy (which frees device memory and therefore waits for the
 * device).  One plan must not be run concurrently from unsynchronised streams. */
typedef struct fasteq_eqlinear_path_c { int32_t input_row, output_row, weight_path, rows; } fasteq_eqlinear_path_c;
typedef struct fasteq_eqlinear_problem_c {
  int32_t B, I, U, P, V, J;              /* batch, rows of x, channels in, paths (= weight blocks), channels out, rows of out */
  const int32_t* i_dims;                 /* host [P]: 2l+1 per path for the dense run-length layout (used when paths is NULL) */
  const fasteq_eqlinear_path_c* paths;   /* host [P] explicit mapping, or NULL */
} fasteq_eqlinear_problem_c;
typedef struct fasteq_eqlinear_plan_info { int32_t precision, forward_impl, dgrad_impl, a_view, j_rows; } fasteq_eqlinear_plan_info;
typedef struct fasteq_eqlinear_backend_api {
  uint32_t abi_version;                  /* 2 */
  int32_t precision;                     /* fasteq_eqlinear_precision */
  int (*forward_create)(const fasteq_eqlinear_problem_c* problem, const void* w, const double* cg /* host [P] */,
                        fasteq_stream_t stream, void** plan, fasteq_eqlinear_plan_info* info /* or NULL */);
  int (*forward_run)(void* plan, const void* x, void* out, fasteq_stream_t stream);
  void (*forward_destroy)(void* plan);
  int (*dgrad_create)(const fasteq_eqlinear_problem_c* problem, const void* w, const double* cg, fasteq_stream_t stream,
                      void** plan, fasteq_eqlinear_plan_info* info);
  int (*dgrad_run)(void* plan, const void* dy, void* dx, fasteq_stream_t stream);
  void (*dgrad_destroy)(void* plan);
  const char* (*status_string)(int code);
} fasteq_eqlinear_backend_api;
const fasteq_eqlinear_backend_api* fasteq_eqlinear_tf32_api(void);
const fasteq_eqlinear_backend_api* fasteq_eqlinear_fp32_api(void);
const fasteq_eqlinear_backend_api* fasteq_eqlinear_fp64_api(void);

/* ------------------------------------------------------------------------- *
 * Gate non-linearity (e3nn nn.Gate) on ir_mul rows [segments, u]: input = scalar segments, one gate
 * segment per gated irrep block, then the gated irreps; output = scalar segments, gated irreps.
 * Activation codes: 0 identity, 1 silu, 2 tanh, 3 sigmoid, 4 abs; cst = the activation's
 * normalisation constant.  Counterpart of fasteq/e3nn/triton/nn/_gate.py:17-39 (a neighbour of the
 * hot path, needed by NequIP-style networks).
 * ------------------------------------------------------------------------- */
typedef struct fasteq_gate_problem {
  int32_t dtype;                /* fasteq_dtype */
  int32_t u;
  int32_t n_scalar, n_gate;
  int64_t batch;
  const int32_t* act;           /* host [n_scalar + n_gate] */
  const double* cst;            /* host [n_scalar + n_gate] */
  const int32_t* gated_dims;    /* host [n_gate] 2l+1 of each gated block */
} fasteq_gate_problem;
int fasteq_gate_forward(const fasteq_gate_problem* p /* host */, const void* x, void* out, fasteq_stream_t stream);
int fasteq_gate_backward(const fasteq_gate_problem* p /* host */, const void* x, const void* grad_out, void* grad_x,
                         fasteq_stream_t stream);
/* Second order: with ggx [batch, n_in, u] the cotangent of grad_x, the gradients of <ggx, grad_x> with respect to
 * grad_out and x (force-loss training through gated networks). */
int fasteq_gate_double_backward(const fasteq_gate_problem* p /* host */, const void* x, const void* grad_out, const void* ggx,
                                void* d_grad_out, void* d_x, fasteq_stream_t stream);

/* Dense layer of the radial MLP: C[M, N] = A[M, K] @ Bt[N, K]^T, FP32 data, 3xTF32 arithmetic on the
 * tensor cores (Bt is a torch.nn.Linear weight, [out_features, in_features]).  K and N multiples of 4,
 * pointers 16-byte aligned, else FASTEQ_UNSUPPORTED.  The reference leaves this MLP to the model
 * package (torch); it has no entry point of its own for it. */
int fasteq_gemm_tf32x3(const void* A, const void* Bt, void* C, int64_t M, int32_t N, int32_t K, fasteq_stream_t stream);
/* The same product with the weight's two TF32 parts prepared beforehand (split holds 2 * N * K floats: hi parts,
 * then lo parts), for weights that stay fixed over many calls. */
int fasteq_gemm_tf32x3_split(const void* Bt, int64_t n_elems, void* split, fasteq_stream_t stream);
int fasteq_gemm_tf32x3_presplit(const void* A, const void* split, void* C, int64_t M, int32_t N, int32_t K, fasteq_stream_t stream);
/* Hidden layers of the radial MLP (width 64, SiLU, no bias) fused into one kernel per direction:
 *   forward : basis [n_edges, n_basis] -> h_1 = silu(W_1 basis) -> ... -> h_L = silu(W_L h_{L-1})
 *   backward: dE/dh_L -> dE/dbasis (weights get no gradient here; train through the layered path)
 * w_first is W_1 [64, n_basis] (n_basis <= 16); w_hidden is a HOST array of n_hidden - 1 device
 * pointers to W_2.. [64, 64] (n_hidden in 1..3).  The first layer runs on the CUDA cores, the 64 x 64
 * layers as 3xTF32 tcgen05 products chained through shared memory and TMEM.  The forward also writes
 * deriv [n_hidden - 1, n_edges, 64] = silu'(z_l) of the tensor-core layers, which the backward reads.
 * out / deriv / grad_out 16-byte aligned.  No counterpart in the reference, which leaves the radial
 * MLP to torch modules of the model package. */
int fasteq_radial_chain_forward(const float* basis, int64_t n_edges, int32_t n_basis, const float* w_first,
                                const float* const* w_hidden /* host */, const float* prepared /* or NULL */, int32_t n_hidden,
                                float* out, float* deriv, fasteq_stream_t stream);
int fasteq_radial_chain_backward(const float* grad_out, const float* deriv, const float* basis, int64_t n_edges,
                                 int32_t n_basis, const float* w_first, const float* const* w_hidden /* host */,
                                 const float* prepared /* or NULL */, int32_t n_hidden, float* grad_basis, fasteq_stream_t stream);
/* The 64 x 64 layers in the form the kernels multiply with (TF32 parts; transposed and in reverse order for the
 * backward): prepared holds (n_hidden - 1) * 2 * 64 * 64 floats and may be passed to the calls above in place
 * of w_hidden while the weights stay unchanged. */
int fasteq_radial_chain_prepare(const float* const* w_hidden /* host */, int32_t n_hidden, int32_t backward, float* prepared,
                                fasteq_stream_t stream);
/* Edge geometry of a radius graph: vec[e] = (pos[src[e]] + shift[e]) - pos[dst[e]] and the radial basis
 * basis[e, n] = sqrt(2 / r_max) sin((n+1) pi r / r_max) / r * env(r / r_max), env the degree-p polynomial cutoff
 * (the embedding of NequIP / MACE models, .../nequip/nn/embedding/_edge.py:174-189, cutoffs.py:17-27; the
 * reference leaves it to torch modules).  The backward takes dE/dvec and / or dE/dbasis (either may be NULL),
 * and overwrites grad_pos [n_nodes, 3] (accumulated with red.global.add over senders and receivers).
 * dtype: fasteq_dtype of pos / shift / vec / basis; n_basis <= 16.  An edge whose sender or receiver index lies
 * outside [0, n_nodes) is not followed: it gets zero features and no gradient, and the status word below reads 2
 * (the tensor-product kernels treat the same index the same way).  A coincident pair (r = 0) gets the limit
 * basis[e, n] = sqrt(2 / r_max) (n+1) pi / r_max and no gradient through the radial basis. */
int fasteq_edge_geometry_forward(int32_t dtype, const void* pos, const int32_t* src, const int32_t* dst, const void* shift,
                                 int64_t n_edges, int64_t n_nodes, double r_max, int32_t n_basis, int32_t envelope_p, void* vec,
                                 void* basis, fasteq_stream_t stream);
int fasteq_edge_geometry_backward(int32_t dtype, const void* pos, const int32_t* src, const int32_t* dst, const void* shift,
                                  const void* grad_vec, const void* grad_basis, int64_t n_edges, int64_t n_nodes, double r_max,
                                  int32_t n_basis, int32_t envelope_p, void* grad_pos, fasteq_stream_t stream);
/* Reads and clears the status word of the edge-geometry kernels (synchronises): 0, or 2 = an edge index was out of range. */
int fasteq_edge_geometry_device_status(int32_t* code /* host */);
/* Reads and clears the status word of the tensor-core kernels (synchronises). */
int fasteq_tensorcore_device_status(int32_t* code /* host */);

#ifdef __cplusplus
}
#endif
#endif /* FASTEQ_B200_H_ */
