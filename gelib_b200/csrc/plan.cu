// Per-device cache of product plans (triple table, band coefficients, work lists).
//
// The reference looks its coefficient matrices up in an unordered_map on every launch and copies
// them to "the" GPU on first use (SO3/SO3CGbank.hpp:33-49, single device only).  Here a plan is
// keyed by (device, kernel family, tiling, part signature), built once under a mutex and kept in
// device memory for the life of the process, so any number of devices can be used from one process.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "plan.h"

namespace gelib_b200 {

std::vector<PartSig> sig_of(const std::vector<PartView>& v) {
  std::vector<PartSig> s;
  for (const auto& p : v) s.push_back({p.l, p.n});
  return s;
}

namespace {
std::mutex g_mu;
std::map<std::vector<int>, DevicePlan*> g_plans;

template <class T>
bool upload(const std::vector<T>& h, T** d) {
  *d = nullptr;
  if (h.empty()) return true;
  if (cudaMalloc((void**)d, h.size() * sizeof(T)) != cudaSuccess) return false;
  return cudaMemcpy(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice) == cudaSuccess;
}
}  // namespace

// ---- options ------------------------------------------------------------------------------------------------

namespace {
struct Options {
  std::atomic<int> fwd{kFwdAuto}, bwd{kBwdAuto}, inject{0}, pair_tma{1}, narrow1{1};
};
int parse_fwd(const char* v) {
  if (!v || !*v || !strcmp(v, "auto")) return kFwdAuto;
  if (!strcmp(v, "simt")) return kFwdSimt;
  if (!strcmp(v, "tcgen05")) return kFwdTc;
  if (!strcmp(v, "tcgen05!")) return kFwdTcStrict;
  return -1;
}
int parse_bwd(const char* v) {
  if (!v || !*v || !strcmp(v, "auto")) return kBwdAuto;
  if (!strcmp(v, "simt")) return kBwdSimt;
  if (!strcmp(v, "pair")) return kBwdPair;
  if (!strcmp(v, "pair!")) return kBwdPairStrict;
  if (!strcmp(v, "tcgen05")) return kBwdTc;
  if (!strcmp(v, "tcgen05!")) return kBwdTcStrict;
  return -1;
}
Options& options() {
  static Options o;
  static std::once_flag once;
  std::call_once(once, [] {
    const int f = parse_fwd(getenv("GELIB_B200_FWD")), b = parse_bwd(getenv("GELIB_B200_BWD"));
    o.fwd = f < 0 ? kFwdAuto : f;
    o.bwd = b < 0 ? kBwdAuto : b;
    const char* inj = getenv("GELIB_B200_INJECT_TIMEOUT");
    o.inject = inj && atoi(inj) != 0;
    const char* tma = getenv("GELIB_B200_PAIR_TMA");
    o.pair_tma = !(tma && !strcmp(tma, "0"));
  });
  return o;
}
}  // namespace

int fwd_mode() { return options().fwd.load(std::memory_order_relaxed); }
int bwd_mode() { return options().bwd.load(std::memory_order_relaxed); }
bool inject_timeout() { return options().inject.load(std::memory_order_relaxed) != 0; }
bool pair_tma() { return options().pair_tma.load(std::memory_order_relaxed) != 0; }
bool narrow1_enabled() { return options().narrow1.load(std::memory_order_relaxed) != 0; }

int set_option(const char* name, const char* value) {
  if (!name) return GELIB_INVALID;
  Options& o = options();
  if (!strcmp(name, "fwd")) {
    const int v = parse_fwd(value);
    if (v < 0) return GELIB_INVALID;
    o.fwd = v;
    return GELIB_OK;
  }
  if (!strcmp(name, "bwd")) {
    const int v = parse_bwd(value);
    if (v < 0) return GELIB_INVALID;
    o.bwd = v;
    return GELIB_OK;
  }
  if (!strcmp(name, "narrow1")) {
    o.narrow1 = !(value && !strcmp(value, "0"));
    return GELIB_OK;
  }
  if (!strcmp(name, "pair_tma")) {
    o.pair_tma = !(value && !strcmp(value, "0"));  // "0": always the cp.async producer; anything else: tensor copies when possible
    return GELIB_OK;
  }
  if (!strcmp(name, "inject_timeout")) {
    o.inject = value && atoi(value) != 0;
    return GELIB_OK;
  }
  return GELIB_INVALID;
}

// ---- status words of kernels with bounded waits --------------------------------------------------------------

namespace {
int* status_words() {
  static int* w = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, kStatusCount * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      w = static_cast<int*>(p);
      for (int i = 0; i < kStatusCount; i++) w[i] = 0;
    } else {
      cudaGetLastError();
    }
  });
  return w;
}
std::atomic<bool> g_status_in_use{false};
}  // namespace

int* async_status_word(int which) {
  int* w = status_words();
  if (!w) return nullptr;
  g_status_in_use.store(true, std::memory_order_relaxed);
  return w + which;
}

int poll_async_status(const char* fn) {
  if (!g_status_in_use.load(std::memory_order_relaxed)) return GELIB_OK;  // no kernel with bounded waits has run yet
  volatile int* w = status_words();
  static const char* what[kStatusCount] = {"the tensor-core forward kernel (cg_fwd_tc_kernel); its output is incomplete",
                                           "the tensor-core backward kernel (cg_bwd_tc_kernel); its gradients are incomplete",
                                           "the backward kernel (cg_bwd_pair_kernel); its gradients are incomplete"};
  std::string msg;
  for (int i = 0; i < kStatusCount; i++)
    if (w[i] != 0) {
      w[i] = 0;
      if (!msg.empty()) msg += "; ";
      msg += what[i];
    }
  if (msg.empty()) return GELIB_OK;
  set_error(std::string(fn) + ": an earlier launch gave up waiting on an mbarrier in " + msg + ".");
  return GELIB_CUDA_ERROR;
}

bool device_has_tcgen05() {
  static std::mutex mu;
  static int cc_major[64];  // 0 = not asked yet, -1 = query failed
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return false;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cc_major[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      cudaGetLastError();
      v = -1;
    }
    cc_major[dev] = v;
  }
  return cc_major[dev] == 10;
}

DevicePlan* get_plan(const std::vector<int>& key, const std::function<void(DevicePlan&)>& build) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error("cudaGetDevice failed");
    return nullptr;
  }
  std::vector<int> k;
  k.push_back(dev);
  k.insert(k.end(), key.begin(), key.end());
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_plans.find(k);
  if (it != g_plans.end()) return it->second;
  DevicePlan* p = new DevicePlan();
  build(*p);
  p->ntriples = (int)p->sched.triples.size();
  p->nitems = (int)p->h_items.size();
  p->njobs = p->h_jobs.empty() ? 0 : (int)p->h_jobs.size() - 1;
  bool ok = upload(p->sched.triples, &p->triples) && upload(p->sched.coeffs, &p->coeffs) &&
            upload(p->h_items, &p->items) && upload(p->h_jobs, &p->jobs) &&
            upload(p->h_floats, &p->floats);
  if (!ok) {
    set_error(std::string("CUDA error while uploading a product plan: ") + cudaGetErrorString(cudaGetLastError()));
    cudaFree(p->triples);
    cudaFree(p->coeffs);
    cudaFree(p->items);
    cudaFree(p->jobs);
    cudaFree(p->floats);
    delete p;
    return nullptr;
  }
  g_plans[k] = p;
  return p;
}

}  // namespace gelib_b200
