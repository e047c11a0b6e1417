// Per-device cache of product plans (triple table, band coefficients, work lists).
//
// The reference looks its coefficient matrices up in an unordered_map on every launch and copies
// them to "the" GPU on first use (SO3/SO3CGbank.hpp:33-49, single device only).  Here a plan is
// keyed by (device, kernel family, tiling, part signature), built once under a mutex and kept in
// device memory for the life of the process, so any number of devices can be used from one process.
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
            upload(p->h_items, &p->items) && upload(p->h_jobs, &p->jobs);
  if (!ok) {
    set_error(std::string("CUDA error while uploading a product plan: ") + cudaGetErrorString(cudaGetLastError()));
    cudaFree(p->triples);
    cudaFree(p->coeffs);
    cudaFree(p->items);
    cudaFree(p->jobs);
    delete p;
    return nullptr;
  }
  g_plans[k] = p;
  return p;
}

}  // namespace gelib_b200
