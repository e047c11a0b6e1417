/*
 * gelib_b200 -- C ABI of the B200 (sm_100a) Clebsch-Gordan kernels.
 *
 * This is the boundary a GElib build binds instead of its own cuda/ directory: every entry
 * point names the reference interface it replaces (paths relative to the GElib source tree).
 * Only plain pointers, sizes and POD descriptors cross it; there are no C++ or torch types.
 *
 * Conventions
 *  - Every SO3part argument is a `gelib_tensor5`: the reference's 5-D canonical form
 *    (batch, grid0, grid1, 2l+1, channels) (core/Gpart.hpp:450-469) of an interleaved
 *    complex-float tensor, with STRIDES IN FLOATS, i.e. twice the complex strides, exactly as
 *    cnine::GPUtensor<float,5> stores them (cuda/GPUtensor.hpp:31-38) but 64-bit so that
 *    tensors beyond 2^31 floats work.  Batch/grid strides may be 0 (broadcast operand,
 *    core/Gpart.hpp:168-185, :366-411).  l is inferred from dims[3] = 2l+1.
 *  - All pointers are device pointers on the CURRENT CUDA device; `stream` is a cudaStream_t
 *    passed as void* (NULL = the default stream).  Calls are asynchronous.
 *  - Outputs are accumulated into (+=), as in the reference (cuda/SO3part_addCGproduct.cu:52-53),
 *    unless GELIB_OVERWRITE is given to a forward call.
 *  - Return value: GELIB_OK, or GELIB_SKIPPED when the reference would GELIB_SKIP (message,
 *    no computation, include/GElib_base.hpp:36), GELIB_INVALID for what the reference turns into
 *    a std::runtime_error (include/GElib_base.hpp:26-33), GELIB_CUDA_ERROR for a CUDA failure.
 *    Nothing throws, exits or traps.  gelib_last_error() returns the calling thread's message.
 */
#ifndef GELIB_B200_H
#define GELIB_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gelib_tensor5 {
  float* base;        /* device pointer to element (0,0,0,0,0) */
  int32_t dims[5];    /* (batch, grid0, grid1, 2l+1, channels) */
  int64_t strides[5]; /* in floats; complex tensors: twice the complex stride */
} gelib_tensor5;

enum { GELIB_OK = 0, GELIB_SKIPPED = 1, GELIB_INVALID = 2, GELIB_CUDA_ERROR = 3 };

/* flags */
enum {
  GELIB_OVERWRITE = 1, /* forward only: the output block is written, not accumulated into, which
                          saves the read-modify-write and the caller's zero fill */
  GELIB_FP64 = 2       /* products and gradients: Clebsch-Gordan coefficients kept in double and every sum accumulated in
                          double, rounded to float once on output.  The reference's bank is single precision only
                          (SO3/SO3CGbank.hpp:52); this is the accuracy path for long accumulations (large l, many
                          channels).  It runs the general strided kernels, at a fraction of the tiled kernels' speed. */
};

#define GELIB_MAX_PARTS 16 /* most parts (distinct l) one SO3vec argument may have */

/* ---- status ---------------------------------------------------------------------------------- */

const char* gelib_version(void);
const char* gelib_last_error(void);          /* message of the last non-OK call of this thread */
const char* gelib_status_string(int status);

/* ---- Clebsch-Gordan coefficients (host) -------------------------------------------------------- */

/* <l1 m1 l2 m2 | l m1+m2>; replaces SO3CGbank::slowCG, SO3/SO3CGbank.hpp:73-95. */
double gelib_CGcoefficient(int l1, int l2, int l, int m1, int m2);
/* Dense (2l1+1) x (2l2+1) float matrix, zero off the band |m1+m2|<=l; replaces
 * SO3CGbank::CGmatrix / get<float>, SO3/SO3CGbank.hpp:33-65.  `out` is host memory. */
int gelib_CGmatrix(int l1, int l2, int l, float* out);

/* ---- type calculus and triple schedule (host) ---------------------------------------------------- */

/* Type of the (Diag)CG product of two SO3vec types; replaces Gtype::CGproduct / DiagCGproduct,
 * core/Gtype.hpp:115-138, with SO3group::for_each_CGcomponent, SO3/SO3group.hpp:43-47.
 * xl/xn (yl/yn): l and channel count of each part.  maxl = -1: no truncation.  Writes up to
 * `cap` (l, n) pairs in ascending l and returns their number (or -1 if cap is too small). */
int gelib_SO3type_CGproduct(int nx, const int* xl, const int* xn, int ny, const int* yl, const int* yn,
                            int maxl, int diag, int cap, int* out_l, int* out_n);

/* The (l1,l2,l,offs) schedule that Gvec::add_CGproduct and its twins walk, core/Gvec.hpp:311-389:
 * l1 ascending, l2 ascending, l = |l1-l2|..l1+l2, skipping l not among rl[], with the running
 * channel offset per output l.  Writes 4 ints per triple into `out` (room for `cap` triples) and
 * returns the number of triples (or -1 if cap is too small). */
int gelib_SO3vec_CGproduct_schedule(int nx, const int* xl, const int* xn, int ny, const int* yl, const int* yn,
                                    int nr, const int* rl, int diag, int cap, int* out);

/* ---- SO3part level: one (l1,l2,l) triple per call ------------------------------------------------- */

/* r[.., m1+m2+l, offs+n1*N2+n2] += C x[.., m1+l1, n1] y[.., m2+l2, n2].
 * Replaces SO3part_addCGproduct_cu, cuda/SO3part_addCGproduct.cu:187-266 (declared SO3/SO3part.hpp:33). */
int gelib_SO3part_addCGproduct(const gelib_tensor5* r, const gelib_tensor5* x, const gelib_tensor5* y,
                               int offs, int flags, void* stream);
/* xg += C g conj(y).  Replaces SO3part_addCGproduct_back0_cu, cuda/SO3part_addCGproduct_back0.cu:224-294
 * (declared SO3/SO3part.hpp:34; argument order (x, r, y) as at core/CGproduct.hpp:81). */
int gelib_SO3part_addCGproduct_back0(const gelib_tensor5* xg, const gelib_tensor5* g, const gelib_tensor5* y,
                                     int offs, int flags, void* stream);
/* yg += C g conj(x).  Replaces SO3part_addCGproduct_back1_cu, cuda/SO3part_addCGproduct_back1.cu:123-175
 * (declared SO3/SO3part.hpp:35; argument order (y, r, x) as at core/CGproduct.hpp:102). */
int gelib_SO3part_addCGproduct_back1(const gelib_tensor5* yg, const gelib_tensor5* g, const gelib_tensor5* x,
                                     int offs, int flags, void* stream);
/* Both gradients from ONE pass over g (what SO3part_CGproductFn.backward needs,
 * python/src/gelib/SO3part.py:188-196).  Equivalent to back0 followed by back1. */
int gelib_SO3part_addCGproduct_back01(const gelib_tensor5* xg, const gelib_tensor5* yg, const gelib_tensor5* g,
                                      const gelib_tensor5* x, const gelib_tensor5* y, int offs, int flags,
                                      void* stream);

/* Diagonal product: channels paired n<->n, output channel offs+n (needs N1 == N2).  These fill in the
 * three GPU routines the reference only declares in comments, SO3/SO3part.hpp:36-38 (its device
 * trampolines SO3/SO3part.hpp:324-334 are empty); semantics = the CPU loops SO3/SO3part.hpp:276-322. */
int gelib_SO3part_addDiagCGproduct(const gelib_tensor5* r, const gelib_tensor5* x, const gelib_tensor5* y,
                                   int offs, int flags, void* stream);
int gelib_SO3part_addDiagCGproduct_back0(const gelib_tensor5* xg, const gelib_tensor5* g, const gelib_tensor5* y,
                                         int offs, int flags, void* stream);
int gelib_SO3part_addDiagCGproduct_back1(const gelib_tensor5* yg, const gelib_tensor5* g, const gelib_tensor5* x,
                                         int offs, int flags, void* stream);
int gelib_SO3part_addDiagCGproduct_back01(const gelib_tensor5* xg, const gelib_tensor5* yg,
                                          const gelib_tensor5* g, const gelib_tensor5* x, const gelib_tensor5* y,
                                          int offs, int flags, void* stream);

/* r += Y_L(x): spherical harmonics of the 3-vectors x (batch,grid0,grid1,3,channels) REAL float tensor
 * (strides in floats), L from r.  Replaces addSPharm_cu, cuda/SPharm.cu:86-123 (declared SO3/SO3part.hpp:39);
 * arithmetic follows the CPU branch SO3/SO3part.hpp:355-394 including the z-axis branch. */
int gelib_SO3part_addSPharm(const gelib_tensor5* r, const gelib_tensor5* x, int flags, void* stream);

/* ---- SO3vec level: all (l1,l2)->l triples in one launch --------------------------------------------- */

/* r_l += sum over triples; parts given as arrays of descriptors, l read from dims[3].
 * Replaces the per-triple launch loop Gvec::add_CGproduct, core/Gvec.hpp:311-321. */
int gelib_SO3vec_addCGproduct(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                              const gelib_tensor5* y, int flags, void* stream);
/* Gvec::add_CGproduct_back0, core/Gvec.hpp:323-333. */
int gelib_SO3vec_addCGproduct_back0(int nx, const gelib_tensor5* xg, int ng, const gelib_tensor5* g, int ny,
                                    const gelib_tensor5* y, int flags, void* stream);
/* Gvec::add_CGproduct_back1, core/Gvec.hpp:335-345. */
int gelib_SO3vec_addCGproduct_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g, int nx,
                                    const gelib_tensor5* x, int flags, void* stream);
/* Both of the above from one pass over g (SO3vec_CGproductFn.backward, python/src/gelib/SO3vec.py:255-270). */
int gelib_SO3vec_addCGproduct_back01(int nx, const gelib_tensor5* xg, int ny, const gelib_tensor5* yg, int ng,
                                     const gelib_tensor5* g, const gelib_tensor5* x, const gelib_tensor5* y,
                                     int flags, void* stream);

/* Diagonal twins: Gvec::add_DiagCGproduct / _back0 / _back1, core/Gvec.hpp:358-389. */
int gelib_SO3vec_addDiagCGproduct(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                                  const gelib_tensor5* y, int flags, void* stream);
int gelib_SO3vec_addDiagCGproduct_back0(int nx, const gelib_tensor5* xg, int ng, const gelib_tensor5* g, int ny,
                                        const gelib_tensor5* y, int flags, void* stream);
int gelib_SO3vec_addDiagCGproduct_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g, int nx,
                                        const gelib_tensor5* x, int flags, void* stream);
int gelib_SO3vec_addDiagCGproduct_back01(int nx, const gelib_tensor5* xg, int ny, const gelib_tensor5* yg,
                                         int ng, const gelib_tensor5* g, const gelib_tensor5* x,
                                         const gelib_tensor5* y, int flags, void* stream);

/* The forward product of gelib_SO3vec_addCGproduct for callers that must not allocate device memory.  (No counterpart
 * in the reference: this entry point exists only here.)
 *
 * Every other product call keeps its tables (triple list, Clebsch-Gordan coefficients) in device memory that the library
 * takes from cudaMalloc the first time it sees a product signature.  Some callers cannot have that: a plug-in that runs
 * inside a framework's memory pool and may not go around it, a service whose device memory has all been handed out
 * before the first request, a latency-bound loop in which cudaMalloc's implicit device synchronisation is not tolerable.
 * This variant runs the general strided kernel with its tables in a fixed 64 KB array that is part of the library image
 * on every GPU that loads it (the memory is held until the process exits, used or not).  It calls no cudaMalloc, no
 * cudaFree and no other allocating routine; inputs and outputs are the caller's, as everywhere else.
 *
 * Limits and rules:
 *  - the product's tables (20 bytes per (l1,l2)->l triple, rounded up to 16, plus 4 bytes per band coefficient) must
 *    fit 65536 bytes, else GELIB_INVALID with the needed size in gelib_last_error() (maxl 6 with 7 parts on either side
 *    needs 34 KB);
 *  - the first call on a device looks the array's device address up (cudaGetSymbolAddress, with that device current);
 *    make that first call outside any stream capture;
 *  - every call uploads its own tables into the shared array on `stream` before its kernel, so calls on one stream are
 *    ordered, but two calls that can overlap on the GPU (different streams or threads) race on the array: serialise them;
 *  - it is the correctness kernel (one thread per output element), not the tiled one: expect a fraction of the speed of
 *    gelib_SO3vec_addCGproduct.
 * Arguments, flags, status codes and results are those of gelib_SO3vec_addCGproduct. */
int gelib_SO3vec_addCGproduct_static(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                                     const gelib_tensor5* y, int flags, void* stream);

/* Spherical harmonics of every part r[i] (any set of l) from one read of x and one Legendre recursion
 * per point; equivalent to one gelib_SO3part_addSPharm call per part (the per-l loop a caller of
 * SO3part.spharm writes, python/src/gelib/SO3part.py:54-62). */
int gelib_SO3vec_addSPharm(int nr, const gelib_tensor5* r, const gelib_tensor5* x, int flags, void* stream);

/* Fused first layer: r (+)= CGproduct(u, y) with u the SO3vec whose part l, l = 0..lmax_x, is the spherical harmonics
 * Y_l(X) in one channel -- the pipeline SO3part.spharm (python/src/gelib/SO3part.py:54-62, SO3/SO3part.hpp:150-156,
 * 340-397) followed by SO3vec CGproduct (core/Gvec.hpp:311-321) -- without the harmonics ever being written to memory:
 * the kernels generate them per point where they stage x.  X: real (batch, 1, 1, 3, 1).  y: parts with one channel count
 * <= 32 and l <= 7 (GELIB_INVALID otherwise).  _back1 is the gradient with respect to y (points carry no gradient):
 * yg += C g conj(u). */
int gelib_SO3vec_addCGproduct_spharm(int nr, const gelib_tensor5* r, const gelib_tensor5* X, int lmax_x, int ny,
                                     const gelib_tensor5* y, int flags, void* stream);
int gelib_SO3vec_addCGproduct_spharm_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g,
                                           const gelib_tensor5* X, int lmax_x, int flags, void* stream);

/* ---- callers of the path ------------------------------------------------------------------------ */

/* Gather along one array dimension of an SO3partArr (message passing): for every outer index o and target t,
 *   r[o][t][:] += sum over k in [row_ptr[t], row_ptr[t+1]) of x[o][col[k]][:]
 * with r (outer, n_out, inner) and x (outer, n_in, inner) dense complex64 tensors and the map as CSR in device memory.
 * Replaces Gpart::add_gather (core/Gpart.hpp:555-557, via cnine::GatherSlices); add_gather_back (core/Gpart.hpp:559-561)
 * is the same call with the transposed map. */
int gelib_add_gather(float* r, const float* x, long long outer, int n_out, int n_in, long long inner, const int* row_ptr,
                     const int* col, void* stream);

/* Channel mixing of a part by a complex weight matrix (all arrays dense complex64, rows = every (cell, m) of the part):
 *   mode 0:  r[row][j] = sum_i x[row][i] W[i][j]            r (rows, n_out), x (rows, n_in), W (n_in, n_out)
 *   mode 1:  r[row][i] = sum_j x[row][j] conj(W[i][j])      r (rows, n_in),  x (rows, n_out): the gradient of the part
 * and the gradient of the weights,  Wg[i][j] += sum_row conj(x[row][i]) g[row][j].  At most 64 channels on either side
 * (GELIB_SKIPPED beyond).  In GElib this is torch.matmul per part (python/src/gelib/SO3vec.py:174-177,
 * python/src/gelib/SO3weights.py:22-85): there is no C++ counterpart. */
int gelib_SO3part_mix(float* r, const float* x, const float* W, long long rows, int n_in, int n_out, int mode, void* stream);
int gelib_SO3part_mix_back_w(float* Wg, const float* x, const float* g, long long rows, int n_in, int n_out, void* stream);

/* Wigner matrix D^l of the rotation with z-y-z Euler angles (alpha, beta, gamma), as SO3irrep::matrix builds it
 * (SO3/SO3irrep.hpp:69-103): out[(m1+l)*(2l+1) + (m2+l)] = d^l_{m2 m1}(beta) e^{i m1 alpha} e^{i m2 gamma}, interleaved
 * (re, im) floats, host memory. */
int gelib_SO3irrep_matrix(int l, double alpha, double beta, double gamma, float* out);

/* r[cell] (+)= D x[cell] for every cell: the rotation of an SO3part (SO3part.apply, python/src/gelib/SO3part.py:132-135,
 * which multiplies by the host-built matrix with torch.matmul).  D: (2l+1)^2 complex64 in DEVICE memory, row-major. */
int gelib_SO3part_apply(const gelib_tensor5* r, const gelib_tensor5* x, const float* D, int flags, void* stream);

/* ---- introspection ------------------------------------------------------------------------------- */

/* Number of kernels this library has launched in the calling process (all threads, all devices). */
long long gelib_kernel_launch_count(void);

/* Measured FP32 multiply-add rate of the current device in TFLOP/s (2 flops per FFMA; best of `reps` launches of a
 * kernel of independent FFMA chains on `ctas` CTAs of 256 threads), the second roof of these kernels beside HBM
 * bandwidth.  `scratch`: ctas*256 floats of the caller's device memory.  <= 0 on failure.  The reference has no
 * counterpart (its benchmark, benchmarking/benchmark_CGproduct.cpp:70-92, reports a CPU op rate). */
double gelib_probe_fp32_tflops(float* scratch, int ctas, int reps, void* stream);

/* Kernel selection and test switches.  The reference chooses between its kernels inside the launcher
 * (cuda/SO3part_addCGproduct.cu:226-262: tiled or not, coefficients preloaded or not) with no way to steer it;
 * here the choice can be pinned.  name "fwd": "auto" | "simt" | "tcgen05" | "tcgen05!";  name "bwd": "auto" |
 * "simt" | "pair" | "pair!" | "tcgen05" | "tcgen05!" (a trailing "!" refuses calls the named kernel cannot take
 * instead of falling back);  name "pair_tma": "1" | "0" (the pair backward kernel fills its ring with tensor copies
 * and the tensor-core forward stores its tiles with tensor copies when the views fit rank-5 tensor maps, "0": cp.async
 * and per-row bulk copies instead);  name "narrow1": "1" | "0" (the
 * gradient of y for a one-channel x takes the kernel written for that shape, "0": the general narrow kernel);
 * name "inject_timeout": "0" | "1" (tests:
 * one bounded device wait is made to run out).
 * Initial values: the environment variables GELIB_B200_FWD, GELIB_B200_BWD, GELIB_B200_PAIR_TMA,
 * GELIB_B200_INJECT_TIMEOUT, read once at first use.  Returns GELIB_OK or GELIB_INVALID. */
int gelib_set_option(const char* name, const char* value);

/* The kernels that wait on mbarriers bound every wait; one that gives up records it in host-mapped memory and
 * returns with incomplete output.  Every product entry point above checks that record first and returns
 * GELIB_CUDA_ERROR for an earlier launch's failure; a caller that wants to know before its next product call
 * synchronises the stream and calls this (GELIB_OK, or GELIB_CUDA_ERROR with the kernel named in
 * gelib_last_error(); the record is cleared).  The reference has no counterpart: its kernels never wait. */
int gelib_async_status(void);

#ifdef __cplusplus
}
#endif
#endif /* GELIB_B200_H */
