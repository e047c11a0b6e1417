// extern "C" entry points: argument validation in the reference's terms, then dispatch to the kernels.
//
// Validation mirrors the host launchers and dispatchers of GElib: the GELIB_SKIP conditions of
// SO3part_addCGproduct_cu (cuda/SO3part_addCGproduct.cu:189-214), the batch/grid reconciliation of
// Gpart_add_CGproduct (core/CGproduct.hpp:44-62, core/Gpart.hpp:168-185, :416-432) and the N1==N2
// assertion of the diagonal loops (SO3/SO3part.hpp:282).
#include <algorithm>
#include <cstring>
#include <map>

#include "plan.h"

using namespace gelib_b200;

namespace {

const char* kVersion = "gelib_b200 0.1 (sm_100a)";

struct Parsed {
  std::vector<PartView> v;  // sorted by l
  std::vector<int> dims0, dims1, dims2;
};

// Converts descriptors to views (sorted by ascending l, as the reference's std::map iterates).
int parse_parts(const char* fn, const char* name, int n, const gelib_tensor5* t, bool real3, std::vector<PartView>* out,
                std::vector<const gelib_tensor5*>* src) {
  if (n < 0 || (n > 0 && !t)) return fail(GELIB_INVALID, fn, std::string("null descriptor array for ") + name);
  if (n > kMaxParts) return fail(GELIB_SKIPPED, fn, std::string(name) + " has more than GELIB_MAX_PARTS parts");
  std::vector<std::pair<int, int>> order;
  for (int i = 0; i < n; i++) {
    bool empty = false;
    for (int d = 0; d < 5; d++) {
      if (t[i].dims[d] < 0) return fail(GELIB_INVALID, fn, std::string("negative dimension in ") + name);
      if (t[i].strides[d] < 0) return fail(GELIB_INVALID, fn, std::string("negative stride in ") + name);
      if (t[i].dims[d] == 0) empty = true;
    }
    if (!t[i].base && !empty) return fail(GELIB_INVALID, fn, std::string("null data pointer in ") + name);
    if (!real3 && !empty) {
      // complex data is read and written as (re, im) pairs with 8-byte accesses
      if ((uintptr_t)t[i].base % 8 != 0)
        return fail(GELIB_INVALID, fn, std::string("data pointer of ") + name + " is not 8-byte aligned");
      for (int d = 0; d < 5; d++)
        if (t[i].dims[d] > 1 && t[i].strides[d] % 2 != 0)
          return fail(GELIB_INVALID, fn, std::string("odd stride (in floats) in complex tensor ") + name);
    }
    if (!real3 && t[i].dims[3] % 2 == 0)
      return fail(GELIB_SKIPPED, fn, std::string("dims[3] of ") + name + " is not of the form 2l+1");
    order.push_back({real3 ? 0 : (t[i].dims[3] - 1) / 2, i});
  }
  std::sort(order.begin(), order.end());
  for (size_t k = 1; k < order.size(); k++)
    if (order[k].first == order[k - 1].first)
      return fail(GELIB_SKIPPED, fn, std::string(name) + " has two parts with the same l");
  out->clear();
  src->clear();
  for (auto& o : order) {
    const gelib_tensor5& d = t[o.second];
    PartView p;
    p.base = d.base;
    p.sb = d.strides[0];
    p.sg0 = d.strides[1];
    p.sg1 = d.strides[2];
    p.sm = d.strides[3];
    p.sc = d.strides[4];
    p.n = d.dims[4];
    p.l = o.first;
    out->push_back(p);
    src->push_back(&d);
  }
  return GELIB_OK;
}

struct Group {
  std::vector<PartView>* v;
  std::vector<const gelib_tensor5*>* src;
  bool* bcast;  // set when a part of the group is broadcast over a dimension the call iterates
};

// Batch and grid reconciliation: every leading dimension is 1 or the call's; 1 becomes stride 0.
int reconcile(const char* fn, std::vector<Group>& groups, CellGrid* cg) {
  int D[3] = {1, 1, 1};
  bool empty[3] = {false, false, false};
  for (auto& g : groups)
    for (auto* s : *g.src)
      for (int d = 0; d < 3; d++) {
        D[d] = std::max(D[d], (int)s->dims[d]);
        if (s->dims[d] == 0) empty[d] = true;
      }
  for (auto& g : groups) {
    for (size_t i = 0; i < g.v->size(); i++) {
      const gelib_tensor5* s = (*g.src)[i];
      PartView& p = (*g.v)[i];
      long long* st[3] = {&p.sb, &p.sg0, &p.sg1};
      for (int d = 0; d < 3; d++) {
        if (empty[d]) continue;
        if (s->dims[d] != D[d] && s->dims[d] != 1)
          return fail(GELIB_SKIPPED, fn, d == 0 ? "batch dimensions cannot be reconciled"
                                                : "grid dimensions cannot be reconciled");
        if (s->dims[d] == 1 && D[d] > 1) *st[d] = 0;
        if (D[d] > 1 && *st[d] == 0 && g.bcast) *g.bcast = true;
      }
    }
  }
  for (int d = 0; d < 3; d++)
    if (empty[d]) D[d] = 0;
  for (int d = 0; d < 3; d++)
    if (D[d] > 65535 && d > 0) return fail(GELIB_SKIPPED, fn, "grid dimension exceeds 65535");
  cg->B = D[0];
  cg->G0 = D[1];
  cg->G1 = D[2];
  cg->ncells = (long long)D[0] * D[1] * D[2];
  return GELIB_OK;
}

bool aligned16(const PartView& p) {
  return ((uintptr_t)p.base % 16 == 0) && p.sb % 4 == 0 && p.sg0 % 4 == 0 && p.sg1 % 4 == 0 && p.sm % 4 == 0;
}

// Checks that every output part has room for the channels the schedule assigns to it.
int check_room(const char* fn, const std::vector<PartView>& x, const std::vector<PartView>& y,
               const std::vector<PartView>& r, bool diag, int offs_extra) {
  Schedule sc;
  build_schedule(sig_of(x), sig_of(y), sig_of(r), diag, false, &sc);
  for (const Triple& t : sc.triples) {
    if (diag && x[t.xi].n != y[t.yi].n)
      return fail(GELIB_INVALID, fn, "failed assertion N1==N2");
    const long long width = diag ? x[t.xi].n : (long long)x[t.xi].n * y[t.yi].n;
    if (t.offs + offs_extra + width > r[t.ri].n)
      return fail(GELIB_SKIPPED, fn, "fragment dimension of r not large enough");
  }
  return GELIB_OK;
}

// mode 0: forward (out = r).  mode 1/2/3: gradient wrt x / y / both (r is g).
int run_product(const char* fn, bool diag, int mode, int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x,
                int ny, const gelib_tensor5* y, int nxg, const gelib_tensor5* xg, int nyg, const gelib_tensor5* yg,
                int offs, int flags, void* stream, bool single_triple, bool no_alloc = false,
                const gelib_tensor5* sph_points = nullptr, int sph_lmax = 0) {
  VecCall c;
  c.diag = diag;
  c.flags = flags;
  c.offs_extra = offs;
  std::vector<const gelib_tensor5*> sr, sx, sy, sxg, syg;
  int st;
  // a kernel of an earlier call whose bounded wait ran out is reported here, whatever this call would run
  if ((st = poll_async_status(fn)) != GELIB_OK) return st;
  if ((st = parse_parts(fn, "r", nr, r, false, &c.r, &sr)) != GELIB_OK) return st;
  if (mode == 0 || mode == 2 || mode == 3)
    if ((st = parse_parts(fn, "x", nx, x, false, &c.x, &sx)) != GELIB_OK) return st;
  if (mode == 0 || mode == 1 || mode == 3)
    if ((st = parse_parts(fn, "y", ny, y, false, &c.y, &sy)) != GELIB_OK) return st;
  if (mode == 1 || mode == 3)
    if ((st = parse_parts(fn, "xg", nxg, xg, false, &c.xg, &sxg)) != GELIB_OK) return st;
  if (mode == 2 || mode == 3)
    if ((st = parse_parts(fn, "yg", nyg, yg, false, &c.yg, &syg)) != GELIB_OK) return st;
  if (offs < 0) return fail(GELIB_SKIPPED, fn, "negative channel offset");

  // a gradient call that does not get the forward operand uses the gradient tensor's shape for it
  if (mode == 1) { c.x = c.xg; sx = sxg; }
  if (mode == 2) { c.y = c.yg; sy = syg; }
  if (mode == 3) {
    if (c.xg.size() != c.x.size() || c.yg.size() != c.y.size())
      return fail(GELIB_INVALID, fn, "gradient vectors must have the parts of x and y");
    for (size_t i = 0; i < c.x.size(); i++)
      if (c.x[i].l != c.xg[i].l || c.x[i].n != c.xg[i].n)
        return fail(GELIB_INVALID, fn, "xg does not have the type of x");
    for (size_t i = 0; i < c.y.size(); i++)
      if (c.y[i].l != c.yg[i].l || c.y[i].n != c.yg[i].n)
        return fail(GELIB_INVALID, fn, "yg does not have the type of y");
  }

  if (single_triple) {
    const int l1 = c.x[0].l, l2 = c.y[0].l, l = c.r[0].l;
    if (l < std::abs(l1 - l2) || l > l1 + l2) return fail(GELIB_SKIPPED, fn, "|l1-l_2| <= l <= l1+l2 not satisfied");
  }

  std::vector<Group> groups;
  groups.push_back({&c.r, &sr, mode == 0 ? &c.r_bcast : nullptr});
  bool dummy = false;
  // in gradient modes 1/2 c.x / c.y alias the gradient view; reconcile the views that are actually used
  if (mode == 0 || mode == 2 || mode == 3) groups.push_back({&c.x, &sx, &dummy});
  if (mode == 0 || mode == 1 || mode == 3) groups.push_back({&c.y, &sy, &dummy});
  if (mode == 1 || mode == 3) groups.push_back({&c.xg, &sxg, &c.xg_bcast});
  if (mode == 2 || mode == 3) groups.push_back({&c.yg, &syg, &c.yg_bcast});
  if ((st = reconcile(fn, groups, &c.cg)) != GELIB_OK) return st;
  if (mode == 1) c.x = c.xg;
  if (mode == 2) c.y = c.yg;

  if ((st = check_room(fn, c.x, c.y, c.r, diag, offs)) != GELIB_OK) return st;

  c.dense_channels = true;
  c.vec_ok = (offs % 2 == 0);
  for (auto* v : {&c.x, &c.y, &c.r, &c.xg, &c.yg})
    for (const auto& p : *v)
      if (p.sc != 2) c.dense_channels = false;
  for (const auto& p : c.r)
    if (!aligned16(p)) c.vec_ok = false;
  for (const auto& p : c.y)
    if (p.n % 2) c.vec_ok = false;
  c.in_vec_ok = true;
  for (auto* v : {&c.x, &c.y, &c.xg, &c.yg})
    for (const auto& p : *v)
      if (!aligned16(p)) c.in_vec_ok = false;
  if (c.cg.ncells == 0) return GELIB_OK;
  if (mode == 0 && c.r_bcast && (flags & GELIB_OVERWRITE))
    return fail(GELIB_INVALID, fn, "GELIB_OVERWRITE with an output that is broadcast over cells (the cells are summed into it)");

  cudaStream_t s = (cudaStream_t)stream;
  if (no_alloc) return launch_cg_strided_static(c, s);
  if (sph_points) {  // fused first layer: the x parts are generated from the points inside the narrow kernels
    c.sph = sph_points->base;
    c.sph_sb = sph_points->dims[0] > 1 ? sph_points->strides[0] : 0;
    c.sph_sm = sph_points->strides[3];
    c.sph_lmax = sph_lmax;
    st = mode == 0 ? launch_cg_narrow_fwd(c, s) : launch_cg_narrow_bwd(c, s);
    if (st == -1)
      return fail(GELIB_INVALID, fn, "the fused spherical-harmonics product takes y parts of one channel count <= 32 with l <= 7");
    return st;
  }
  const bool fp64 = (flags & GELIB_FP64) != 0;  // double coefficients and sums: the general strided kernels
  if (mode == 0) {
    st = -1;
    if (c.dense_channels && !c.r_bcast && !fp64) {
      if (diag) {
        st = launch_diag_fwd(c, s);
      } else {
        st = launch_cg_narrow_fwd(c, s);
        if (st == -1) st = launch_cg_fwd(c, s);
      }
    }
    if (st == -1) st = launch_cg_strided(c, 0, s);
    return st;
  }
  st = -1;
  if (c.dense_channels && !fp64) {
    if (diag) {
      st = launch_diag_bwd(c, s);
    } else {
      st = launch_cg_narrow_bwd(c, s);
      if (st == -1) st = launch_cg_bwd(c, s);
    }
  }
  if (st == -1) {
    st = GELIB_OK;
    if (!c.xg.empty()) st = launch_cg_strided(c, 1, s);
    if (st == GELIB_OK && !c.yg.empty()) st = launch_cg_strided(c, 2, s);
  }
  return st;
}

int type_product(int nx, const int* xl, const int* xn, int ny, const int* yl, const int* yn, int maxl, bool diag,
                 std::map<int, long long>* out) {
  std::vector<std::pair<int, int>> xs, ys;
  for (int i = 0; i < nx; i++) xs.push_back({xl[i], xn[i]});
  for (int i = 0; i < ny; i++) ys.push_back({yl[i], yn[i]});
  std::sort(xs.begin(), xs.end());
  std::sort(ys.begin(), ys.end());
  for (auto& p : xs)
    for (auto& q : ys)
      for (int l = std::abs(p.first - q.first); l <= p.first + q.first; l++)
        if (maxl == -1 || l <= maxl) (*out)[l] += diag ? p.second : (long long)p.second * q.second;
  return 0;
}

}  // namespace

extern "C" {

const char* gelib_version(void) { return kVersion; }
const char* gelib_last_error(void) { return last_error().c_str(); }
const char* gelib_status_string(int status) {
  switch (status) {
    case GELIB_OK: return "ok";
    case GELIB_SKIPPED: return "skipped: arguments the reference would GELIB_SKIP";
    case GELIB_INVALID: return "invalid arguments";
    case GELIB_CUDA_ERROR: return "CUDA error";
    default: return "unknown status";
  }
}

double gelib_CGcoefficient(int l1, int l2, int l, int m1, int m2) { return cg_coefficient(l1, l2, l, m1, m2); }

int gelib_CGmatrix(int l1, int l2, int l, float* out) {
  static const char* fn = "gelib_CGmatrix";
  if (!out) return fail(GELIB_INVALID, fn, "null output");
  if (l1 < 0 || l2 < 0 || l < std::abs(l1 - l2) || l > l1 + l2)
    return fail(GELIB_SKIPPED, fn, "|l1-l_2| <= l <= l1+l2 not satisfied");
  const int L2 = 2 * l2 + 1;
  for (int m1 = -l1; m1 <= l1; m1++)
    for (int m2 = -l2; m2 <= l2; m2++)
      out[(m1 + l1) * L2 + (m2 + l2)] = std::abs(m1 + m2) <= l ? (float)cg_coefficient(l1, l2, l, m1, m2) : 0.f;
  return GELIB_OK;
}

int gelib_SO3type_CGproduct(int nx, const int* xl, const int* xn, int ny, const int* yl, const int* yn, int maxl,
                            int diag, int cap, int* out_l, int* out_n) {
  if (nx < 0 || ny < 0 || cap < 0 || (nx > 0 && (!xl || !xn)) || (ny > 0 && (!yl || !yn)) || (cap > 0 && (!out_l || !out_n)))
    return -2;
  for (int i = 0; i < nx; i++) if (xl[i] < 0 || xn[i] < 0) return -2;
  for (int i = 0; i < ny; i++) if (yl[i] < 0 || yn[i] < 0) return -2;
  std::map<int, long long> R;
  type_product(nx, xl, xn, ny, yl, yn, maxl, diag != 0, &R);
  if ((int)R.size() > cap) return -1;
  int k = 0;
  for (auto& p : R) {
    out_l[k] = p.first;
    out_n[k] = (int)p.second;
    k++;
  }
  return k;
}

int gelib_SO3vec_CGproduct_schedule(int nx, const int* xl, const int* xn, int ny, const int* yl, const int* yn, int nr,
                                    const int* rl, int diag, int cap, int* out) {
  if (nx < 0 || ny < 0 || nr < 0 || cap < 0 || (nx > 0 && (!xl || !xn)) || (ny > 0 && (!yl || !yn)) || (nr > 0 && !rl) ||
      (cap > 0 && !out))
    return -2;
  for (int i = 0; i < nx; i++) if (xl[i] < 0 || xn[i] < 0) return -2;
  for (int i = 0; i < ny; i++) if (yl[i] < 0 || yn[i] < 0) return -2;
  for (int i = 0; i < nr; i++) if (rl[i] < 0) return -2;
  std::vector<PartSig> xs, ys, rs;
  for (int i = 0; i < nx; i++) xs.push_back({xl[i], xn[i]});
  for (int i = 0; i < ny; i++) ys.push_back({yl[i], yn[i]});
  for (int i = 0; i < nr; i++) rs.push_back({rl[i], 0});
  auto by_l = [](const PartSig& a, const PartSig& b) { return a.l < b.l; };
  std::sort(xs.begin(), xs.end(), by_l);
  std::sort(ys.begin(), ys.end(), by_l);
  std::sort(rs.begin(), rs.end(), by_l);
  Schedule sc;
  build_schedule(xs, ys, rs, diag != 0, false, &sc);
  if ((int)sc.triples.size() > cap) return -1;
  for (size_t i = 0; i < sc.triples.size(); i++) {
    out[4 * i + 0] = sc.triples[i].l1;
    out[4 * i + 1] = sc.triples[i].l2;
    out[4 * i + 2] = sc.triples[i].l;
    out[4 * i + 3] = sc.triples[i].offs;
  }
  return (int)sc.triples.size();
}

// ---- SO3part level ---------------------------------------------------------------------------------------

int gelib_SO3part_addCGproduct(const gelib_tensor5* r, const gelib_tensor5* x, const gelib_tensor5* y, int offs,
                               int flags, void* stream) {
  return run_product("SO3part_addCGproduct", false, 0, 1, r, 1, x, 1, y, 0, nullptr, 0, nullptr, offs, flags, stream, true);
}
int gelib_SO3part_addCGproduct_back0(const gelib_tensor5* xg, const gelib_tensor5* g, const gelib_tensor5* y, int offs,
                                     int flags, void* stream) {
  return run_product("SO3part_addCGproduct_back0", false, 1, 1, g, 0, nullptr, 1, y, 1, xg, 0, nullptr, offs, flags, stream, true);
}
int gelib_SO3part_addCGproduct_back1(const gelib_tensor5* yg, const gelib_tensor5* g, const gelib_tensor5* x, int offs,
                                     int flags, void* stream) {
  return run_product("SO3part_addCGproduct_back1", false, 2, 1, g, 1, x, 0, nullptr, 0, nullptr, 1, yg, offs, flags, stream, true);
}
int gelib_SO3part_addCGproduct_back01(const gelib_tensor5* xg, const gelib_tensor5* yg, const gelib_tensor5* g,
                                      const gelib_tensor5* x, const gelib_tensor5* y, int offs, int flags,
                                      void* stream) {
  return run_product("SO3part_addCGproduct_back01", false, 3, 1, g, 1, x, 1, y, 1, xg, 1, yg, offs, flags, stream, true);
}

int gelib_SO3part_addDiagCGproduct(const gelib_tensor5* r, const gelib_tensor5* x, const gelib_tensor5* y, int offs,
                                   int flags, void* stream) {
  return run_product("SO3part_addDiagCGproduct", true, 0, 1, r, 1, x, 1, y, 0, nullptr, 0, nullptr, offs, flags, stream, true);
}
int gelib_SO3part_addDiagCGproduct_back0(const gelib_tensor5* xg, const gelib_tensor5* g, const gelib_tensor5* y,
                                         int offs, int flags, void* stream) {
  return run_product("SO3part_addDiagCGproduct_back0", true, 1, 1, g, 0, nullptr, 1, y, 1, xg, 0, nullptr, offs, flags, stream, true);
}
int gelib_SO3part_addDiagCGproduct_back1(const gelib_tensor5* yg, const gelib_tensor5* g, const gelib_tensor5* x,
                                         int offs, int flags, void* stream) {
  return run_product("SO3part_addDiagCGproduct_back1", true, 2, 1, g, 1, x, 0, nullptr, 0, nullptr, 1, yg, offs, flags, stream, true);
}
int gelib_SO3part_addDiagCGproduct_back01(const gelib_tensor5* xg, const gelib_tensor5* yg, const gelib_tensor5* g,
                                          const gelib_tensor5* x, const gelib_tensor5* y, int offs, int flags,
                                          void* stream) {
  return run_product("SO3part_addDiagCGproduct_back01", true, 3, 1, g, 1, x, 1, y, 1, xg, 1, yg, offs, flags, stream, true);
}

// ---- SO3vec level ----------------------------------------------------------------------------------------

int gelib_SO3vec_addCGproduct(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                              const gelib_tensor5* y, int flags, void* stream) {
  return run_product("SO3vec_addCGproduct", false, 0, nr, r, nx, x, ny, y, 0, nullptr, 0, nullptr, 0, flags, stream, false);
}
int gelib_SO3vec_addCGproduct_back0(int nx, const gelib_tensor5* xg, int ng, const gelib_tensor5* g, int ny,
                                    const gelib_tensor5* y, int flags, void* stream) {
  return run_product("SO3vec_addCGproduct_back0", false, 1, ng, g, 0, nullptr, ny, y, nx, xg, 0, nullptr, 0, flags, stream, false);
}
int gelib_SO3vec_addCGproduct_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g, int nx,
                                    const gelib_tensor5* x, int flags, void* stream) {
  return run_product("SO3vec_addCGproduct_back1", false, 2, ng, g, nx, x, 0, nullptr, 0, nullptr, ny, yg, 0, flags, stream, false);
}
int gelib_SO3vec_addCGproduct_back01(int nx, const gelib_tensor5* xg, int ny, const gelib_tensor5* yg, int ng,
                                     const gelib_tensor5* g, const gelib_tensor5* x, const gelib_tensor5* y, int flags,
                                     void* stream) {
  return run_product("SO3vec_addCGproduct_back01", false, 3, ng, g, nx, x, ny, y, nx, xg, ny, yg, 0, flags, stream, false);
}

int gelib_SO3vec_addDiagCGproduct(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                                  const gelib_tensor5* y, int flags, void* stream) {
  return run_product("SO3vec_addDiagCGproduct", true, 0, nr, r, nx, x, ny, y, 0, nullptr, 0, nullptr, 0, flags, stream, false);
}
int gelib_SO3vec_addDiagCGproduct_back0(int nx, const gelib_tensor5* xg, int ng, const gelib_tensor5* g, int ny,
                                        const gelib_tensor5* y, int flags, void* stream) {
  return run_product("SO3vec_addDiagCGproduct_back0", true, 1, ng, g, 0, nullptr, ny, y, nx, xg, 0, nullptr, 0, flags, stream, false);
}
int gelib_SO3vec_addDiagCGproduct_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g, int nx,
                                        const gelib_tensor5* x, int flags, void* stream) {
  return run_product("SO3vec_addDiagCGproduct_back1", true, 2, ng, g, nx, x, 0, nullptr, 0, nullptr, ny, yg, 0, flags, stream, false);
}
int gelib_SO3vec_addDiagCGproduct_back01(int nx, const gelib_tensor5* xg, int ny, const gelib_tensor5* yg, int ng,
                                         const gelib_tensor5* g, const gelib_tensor5* x, const gelib_tensor5* y,
                                         int flags, void* stream) {
  return run_product("SO3vec_addDiagCGproduct_back01", true, 3, ng, g, nx, x, ny, y, nx, xg, ny, yg, 0, flags, stream, false);
}

int gelib_SO3vec_addCGproduct_static(int nr, const gelib_tensor5* r, int nx, const gelib_tensor5* x, int ny,
                                     const gelib_tensor5* y, int flags, void* stream) {
  return run_product("SO3vec_addCGproduct_static", false, 0, nr, r, nx, x, ny, y, 0, nullptr, 0, nullptr, 0, flags, stream, false,
                     true);
}

// ---- fused first layer: r = CG(Y_0..lmax(X), y) without the harmonics ever reaching memory ------------------------

namespace {
int run_sph_product(const char* fn, int mode, int nr, const gelib_tensor5* r, const gelib_tensor5* X, int lmax_x, int ny,
                    const gelib_tensor5* y, int flags, void* stream) {
  if (!X || !X->base) return fail(GELIB_INVALID, fn, "null points");
  if (lmax_x < 0 || lmax_x >= GELIB_MAX_PARTS) return fail(GELIB_SKIPPED, fn, "lmax of the harmonics out of range");
  if (X->dims[3] != 3 || X->dims[4] != 1 || X->dims[1] != 1 || X->dims[2] != 1)
    return fail(GELIB_SKIPPED, fn, "points must be (batch, 3, 1)");
  // stand-in descriptors for the harmonics: right shapes, never dereferenced (the kernels generate the values)
  gelib_tensor5 xd[GELIB_MAX_PARTS];
  for (int l = 0; l <= lmax_x; l++) {
    xd[l].base = reinterpret_cast<float*>(reinterpret_cast<uintptr_t>(X->base) & ~(uintptr_t)7);
    const int dims[5] = {X->dims[0], 1, 1, 2 * l + 1, 1};
    for (int d = 0; d < 5; d++) {
      xd[l].dims[d] = dims[d];
      xd[l].strides[d] = d >= 3 ? 2 : 0;  // dense in the channel, as the kernels' qualification wants
    }
  }
  if (mode == 0)
    return run_product(fn, false, 0, nr, r, lmax_x + 1, xd, ny, y, 0, nullptr, 0, nullptr, 0, flags, stream, false, false, X, lmax_x);
  return run_product(fn, false, 2, nr, r, lmax_x + 1, xd, 0, nullptr, 0, nullptr, ny, y, 0, flags, stream, false, false, X, lmax_x);
}
}  // namespace

int gelib_SO3vec_addCGproduct_spharm(int nr, const gelib_tensor5* r, const gelib_tensor5* X, int lmax_x, int ny,
                                     const gelib_tensor5* y, int flags, void* stream) {
  return run_sph_product("SO3vec_addCGproduct_spharm", 0, nr, r, X, lmax_x, ny, y, flags, stream);
}
int gelib_SO3vec_addCGproduct_spharm_back1(int ny, const gelib_tensor5* yg, int ng, const gelib_tensor5* g,
                                           const gelib_tensor5* X, int lmax_x, int flags, void* stream) {
  return run_sph_product("SO3vec_addCGproduct_spharm_back1", 2, ng, g, X, lmax_x, ny, yg, flags, stream);
}

// ---- spherical harmonics ------------------------------------------------------------------------------------

int gelib_SO3vec_addSPharm(int nr, const gelib_tensor5* r, const gelib_tensor5* x, int flags, void* stream) {
  static const char* fn = "addSPharm";
  VecCall c;
  std::vector<const gelib_tensor5*> sr, sx;
  std::vector<PartView> xv;
  int st;
  if ((st = parse_parts(fn, "r", nr, r, false, &c.r, &sr)) != GELIB_OK) return st;
  if ((st = parse_parts(fn, "x", 1, x, true, &xv, &sx)) != GELIB_OK) return st;
  if (x->dims[3] != 3) return fail(GELIB_SKIPPED, fn, "dim(-2) of x must be 3");
  for (const auto& p : c.r)
    if (p.n != xv[0].n) return fail(GELIB_INVALID, fn, "channel dimensions of x and r differ");
  std::vector<Group> groups;
  bool rb = false, xb = false;
  groups.push_back({&c.r, &sr, &rb});
  groups.push_back({&xv, &sx, &xb});
  if ((st = reconcile(fn, groups, &c.cg)) != GELIB_OK) return st;
  if (rb) return fail(GELIB_SKIPPED, fn, "r is broadcast over the batch");
  return launch_spharm(c.r, xv[0], c.cg, flags, (cudaStream_t)stream);
}

int gelib_SO3part_addSPharm(const gelib_tensor5* r, const gelib_tensor5* x, int flags, void* stream) {
  return gelib_SO3vec_addSPharm(1, r, x, flags, stream);
}

// ---- callers of the path: gather over an array dimension, Wigner-D apply --------------------------------------

int gelib_add_gather(float* r, const float* x, long long outer, int n_out, int n_in, long long inner, const int* row_ptr,
                     const int* col, void* stream) {
  static const char* fn = "add_gather";
  if (outer < 0 || n_out < 0 || n_in < 0 || inner < 0) return fail(GELIB_INVALID, fn, "negative size");
  if ((outer && n_out && inner) && (!r || !x || !row_ptr || !col)) return fail(GELIB_INVALID, fn, "null pointer");
  return launch_gather(r, x, outer, n_out, n_in, inner, row_ptr, col, (cudaStream_t)stream);
}

int gelib_SO3part_mix(float* r, const float* x, const float* W, long long rows, int n_in, int n_out, int mode, void* stream) {
  static const char* fn = "SO3part_mix";
  if (rows < 0 || n_in < 0 || n_out < 0 || (mode != 0 && mode != 1)) return fail(GELIB_INVALID, fn, "negative size or unknown mode");
  if (rows && (!r || !x || !W)) return fail(GELIB_INVALID, fn, "null pointer");
  if ((reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) % 8)
    return fail(GELIB_INVALID, fn, "complex arrays must be 8-byte aligned");
  return launch_mix(r, x, W, rows, n_in, n_out, mode, (cudaStream_t)stream);
}

int gelib_SO3part_mix_back_w(float* Wg, const float* x, const float* g, long long rows, int n_in, int n_out, void* stream) {
  static const char* fn = "SO3part_mix_back_w";
  if (rows < 0 || n_in < 0 || n_out < 0) return fail(GELIB_INVALID, fn, "negative size");
  if (rows && (!Wg || !x || !g)) return fail(GELIB_INVALID, fn, "null pointer");
  if ((reinterpret_cast<uintptr_t>(Wg) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g)) % 8)
    return fail(GELIB_INVALID, fn, "complex arrays must be 8-byte aligned");
  return launch_mix_back_w(Wg, x, g, rows, n_in, n_out, (cudaStream_t)stream);
}

int gelib_SO3irrep_matrix(int l, double alpha, double beta, double gamma, float* out) {
  if (l < 0 || !out) return fail(GELIB_INVALID, "SO3irrep_matrix", "negative l or null output");
  wigner_D(l, alpha, beta, gamma, out);
  return GELIB_OK;
}

int gelib_SO3part_apply(const gelib_tensor5* r, const gelib_tensor5* x, const float* D, int flags, void* stream) {
  static const char* fn = "SO3part_apply";
  VecCall c;
  std::vector<const gelib_tensor5*> sr, sx;
  std::vector<PartView> xv;
  int st;
  if (!D) return fail(GELIB_INVALID, fn, "null matrix");
  if ((st = parse_parts(fn, "r", 1, r, false, &c.r, &sr)) != GELIB_OK) return st;
  if ((st = parse_parts(fn, "x", 1, x, false, &xv, &sx)) != GELIB_OK) return st;
  if (c.r[0].l != xv[0].l || c.r[0].n != xv[0].n) return fail(GELIB_INVALID, fn, "r does not have the shape of x");
  std::vector<Group> groups;
  bool rb = false, xb = false;
  groups.push_back({&c.r, &sr, &rb});
  groups.push_back({&xv, &sx, &xb});
  if ((st = reconcile(fn, groups, &c.cg)) != GELIB_OK) return st;
  if (rb) return fail(GELIB_SKIPPED, fn, "r is broadcast over the batch");
  return launch_apply(c.r[0], xv[0], c.cg, D, flags, (cudaStream_t)stream);
}

long long gelib_kernel_launch_count(void) { return launch_count(); }

int gelib_set_option(const char* name, const char* value) {
  const int st = set_option(name, value);
  if (st != GELIB_OK) return fail(GELIB_INVALID, "gelib_set_option", "unknown option name or value");
  return GELIB_OK;
}

double gelib_probe_fp32_tflops(float* scratch, int ctas, int reps, void* stream) {
  return probe_fp32_tflops(scratch, ctas, reps, (cudaStream_t)stream);
}

int gelib_async_status(void) { return poll_async_status("gelib_async_status"); }

}  // extern "C"
