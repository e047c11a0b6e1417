// Host-side description of one product call and the per-device plan cache.
#pragma once
#include <functional>
#include <vector>

#include "common.h"

namespace gelib_b200 {

// A validated vector-level product.  For the forward pass `r` is the output; for the backward
// passes `r` holds the upstream gradient g and xg / yg the requested outputs (either may be empty).
struct VecCall {
  std::vector<PartView> x, y, r, xg, yg;
  CellGrid cg;
  bool diag = false;
  int offs_extra = 0;    // added to every triple's channel offset (the `offs` of the SO3part-level calls)
  int flags = 0;
  bool r_bcast = false;  // an output tensor is broadcast over cells: results must be summed (atomics)
  bool xg_bcast = false, yg_bcast = false;
  bool dense_channels = true;  // every tensor has channel stride 2 floats
  bool vec_ok = true;          // 16-byte alignment of bases/strides/offsets of r (g) holds, offsets and n2 even
  const float* sph = nullptr;  // fused first layer: x parts are the harmonics of these points (cell, 3), never read
  long long sph_sb = 0, sph_sm = 0;
  int sph_lmax = 0;
  bool in_vec_ok = true;       // 16-byte alignment of every x, y, xg, yg part (float4 access to the small operands)
};

std::vector<PartSig> sig_of(const std::vector<PartView>& v);

// Returns the cached plan for `key` on the current device, building and uploading it on first use.
// `build` fills sched / h_items / h_jobs.  nullptr (with the error message set) on CUDA failure.
DevicePlan* get_plan(const std::vector<int>& key, const std::function<void(DevicePlan&)>& build);

// Kernel families (each returns a status code).
int launch_cg_fwd(const VecCall& c, cudaStream_t s);
int launch_cg_fwd_tc(const VecCall& c, cudaStream_t s, int min_slabs);  // tcgen05 kernel; -1 when the call does not qualify or has fewer slabs per cell
int launch_cg_bwd(const VecCall& c, cudaStream_t s);
int launch_cg_bwd_tc(const VecCall& c, cudaStream_t s);  // tcgen05 kernel; -1 when the call does not qualify
int launch_cg_bwd_pair(const VecCall& c, cudaStream_t s, int min_groups);  // uncoupled-gradient kernel; -1 when the call does not qualify or has fewer groups per cell
int launch_cg_narrow_bwd(const VecCall& c, cudaStream_t s);
int launch_cg_narrow1_bwd(const VecCall& c, cudaStream_t s);  // x with one channel, gradient of y only; -1 otherwise
bool narrow1_enabled();  // option "narrow1" (default on): tests compare the two kernels
int launch_cg_narrow_fwd(const VecCall& c, cudaStream_t s);  // x with at most 4 channels; -1 when the call does not qualify
int launch_cg_strided(const VecCall& c, int mode, cudaStream_t s);  // mode 0 fwd, 1 back0, 2 back1
int launch_cg_strided_static(const VecCall& c, cudaStream_t s);  // forward, tables in a static device array: no allocation
int launch_diag_fwd(const VecCall& c, cudaStream_t s);
int launch_diag_bwd(const VecCall& c, cudaStream_t s);
int launch_diag_fwd_fast(const VecCall& c, cudaStream_t s);  // -1 when the call does not qualify
int launch_diag_bwd_fast(const VecCall& c, cudaStream_t s);  // -1 when the call does not qualify
// Work items of a diagonal product (defined in diag.cu): {first triple | nl<<16, m, coefficient offset, padded nl}
void build_diag_items(DevicePlan& p, const std::vector<PartSig>& xs, const std::vector<PartSig>& ys,
                      const std::vector<PartSig>& rs, int* max_nl);
int launch_gather(float* r, const float* x, long long outer, int n_out, int n_in, long long inner, const int* row_ptr,
                  const int* col, cudaStream_t s);
int launch_mix(float* r, const float* x, const float* W, long long rows, int n_in, int n_out, int mode, cudaStream_t s);
int launch_mix_back_w(float* Wg, const float* x, const float* g, long long rows, int n_in, int n_out, cudaStream_t s);
int launch_apply(const PartView& r, const PartView& x, const CellGrid& cg, const float* D, int flags, cudaStream_t s);
void wigner_D(int l, double alpha, double beta, double gamma, float* out);
int launch_spharm(const std::vector<PartView>& r, const PartView& x, const CellGrid& cg, int flags, cudaStream_t s);

// Kernel selection and debug switches.  Initial values come from the environment (GELIB_B200_FWD, GELIB_B200_BWD,
// GELIB_B200_INJECT_TIMEOUT), read once at first use; gelib_set_option changes them afterwards.  Launch paths read
// one atomic integer.
enum FwdMode { kFwdAuto = 0, kFwdSimt, kFwdTc, kFwdTcStrict };
enum BwdMode { kBwdAuto = 0, kBwdSimt, kBwdPair, kBwdPairStrict, kBwdTc, kBwdTcStrict };
int fwd_mode();
int bwd_mode();
bool pair_tma();        // the pair backward kernel fills its ring with tensor copies when the views allow (default on)
bool inject_timeout();  // tests only: make one bounded device wait run out (no fault is involved)
int set_option(const char* name, const char* value);  // GELIB_OK or GELIB_INVALID

// Host-mapped status words that kernels with bounded waits set when a wait ran out.  One word per kernel family;
// every C-ABI product call and gelib_async_status() poll and clear them.
enum { kStatusFwdTc = 0, kStatusBwdTc = 1, kStatusBwdPair = 2, kStatusCount = 3 };
int* async_status_word(int which);        // nullptr when the mapped allocation failed
int poll_async_status(const char* fn);    // GELIB_OK, or GELIB_CUDA_ERROR with the message set (words cleared)

double probe_fp32_tflops(float* scratch, int ctas, int reps, cudaStream_t s);  // measured FFMA rate, probe.cu
bool device_has_tcgen05();  // compute capability 10.x on the current device (cached per device)
long long launch_count();
const std::string& last_error();

}  // namespace gelib_b200
