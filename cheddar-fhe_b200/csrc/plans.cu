// Per-level constants of ModUp / ModDown / Rescale / ModDownAndRescale, built
// once at context creation (the reference builds one ModSwitchHandler per
// level, src/core/ModSwitch.cu:175-318, with constants from :320-411).
#include <algorithm>
#include <cstdlib>
#include <string>

#include "context.h"
#include "host_math.h"
#include "kernels.h"

namespace cfhe {
namespace {

uint32_t prod_mod(const Context &c, const std::vector<int> &gs, uint32_t p,
                  int skip = -1) {
  uint32_t acc = 1;
  for (int j = 0; j < (int)gs.size(); j++)
    if (j != skip) acc = mulmod(acc, c.q[gs[j]] % p, p);
  return acc;
}

int32_t centre(uint32_t a, uint32_t q) {
  return a > (q >> 1) ? (int32_t)(a - q) : (int32_t)a;
}

// Fills pre-scale constants and the device table of S -> D.
int finish_conv(const Context &c, ConvPlan &cv, const std::vector<int> &restored) {
  const int ns = cv.src_g.size(), nd = cv.dst_g.size();
  cv.pre.resize(ns);
  for (int k = 0; k < ns; k++) {
    const uint32_t s = c.q[cv.src_g[k]];
    uint32_t v = prod_mod(c, cv.src_g, s, k);
    v = mulmod(v, (uint32_t)c.n % s, s);
    v = invmod(v, s);
    v = mulmod(v, prod_mod(c, restored, s), s);
    cv.pre[k] = v;
  }
  std::vector<int32_t> t((size_t)ns * nd);
  for (int m = 0; m < nd; m++) {
    const uint32_t p = c.q[cv.dst_g[m]];
    for (int k = 0; k < ns; k++)
      t[(size_t)m * ns + k] =
          centre(to_mont(to_mont(prod_mod(c, cv.src_g, p, k), p), p), p);
  }
  CFHE_CUDA(cudaMalloc(&cv.d_table, t.size() * sizeof(int32_t)));
  CFHE_CUDA(cudaMemcpy(cv.d_table, t.data(), t.size() * sizeof(int32_t),
                       cudaMemcpyHostToDevice));
  for (size_t k = 0; k < cv.pre.size(); k++) {
    const uint32_t q = c.q[cv.src_g[k]];
    cv.pre_tw.push_back(make_tw(mulmod(cv.pre[k] % q, rinv_mod(q), q), q));
  }
  for (size_t m = 0; m < cv.ep_pad.size(); m++) {
    const uint32_t q = c.q[cv.dst_g[m]];
    cv.ep_pad_tw.push_back(make_tw(cv.ep_pad[m], q));
    cv.ep_scale_tw.push_back(make_tw(cv.ep_scale[m], q));
    cv.ep_ps_tw.push_back(make_tw(mulmod(cv.ep_pad[m] % q, cv.ep_scale[m] % q, q), q));
  }
  return build_tc_table(c, cv);
}

void np_limbs(const Context &c, int nm, int nt, int na, std::vector<int> &g) {
  g.clear();
  for (int i = c.T - nt; i < c.T + nm; i++) g.push_back(i);
  for (int a = 0; a < na; a++) g.push_back(c.L + a);
}

// Source limbs `src` (global indices, in storage order) are switched to the
// Q limbs `dst`: limbs of src that are not in dst form S, limbs of dst that
// are not in src are "restored" (rational rescaling).
int build_down(const Context &c, ConvPlan &cv, const std::vector<int> &src,
               const std::vector<int> &dst) {
  std::vector<int> restored;
  for (int k = 0; k < (int)src.size(); k++)
    if (std::find(dst.begin(), dst.end(), src[k]) == dst.end()) {
      cv.src_g.push_back(src[k]);
      cv.src_pos.push_back(k);
    }
  for (int g : dst)
    if (std::find(src.begin(), src.end(), g) == src.end()) restored.push_back(g);
  cv.dst_g = dst;
  cv.has_pad = !restored.empty();
  for (int g : dst) {
    const uint32_t p = c.q[g];
    auto it = std::find(src.begin(), src.end(), g);
    cv.ep_pos.push_back(it == src.end() ? -1 : (int)(it - src.begin()));
    cv.ep_pad.push_back(prod_mod(c, restored, p));
    cv.ep_scale.push_back(invmod(prod_mod(c, cv.src_g, p), p));
  }
  return finish_conv(c, cv, restored);
}

}  // namespace

int build_plans(Context &c) {
  const char *mode = getenv("CFHE_BCONV");
  c.use_tc_bconv = !(mode && std::string(mode) == "simt");
  const char *lt = getenv("CFHE_LT");
  c.use_fused_lt = !(lt && std::string(lt) == "unfused");
  const char *pdl = getenv("CFHE_PDL");
  c.use_pdl = !(pdl && std::string(pdl) == "0");
  const char *ntt_mode = getenv("CFHE_NTT");
  c.use_twopass_ntt = !(ntt_mode && std::string(ntt_mode) == "cluster");
  // CFHE_NTT: "tiled" = always the pipelined kernels, "twopass" / "cluster" = never, otherwise by shape
  c.ntt_policy = !ntt_mode ? 1 : std::string(ntt_mode) == "tiled" ? 2 : 0;
  {
    const char *chunk = getenv("CFHE_NTT_CHUNK");
    const char *unit = getenv("CFHE_NTT_UNIT");
    c.ntt_chunk = chunk ? atoi(chunk) : 640;
    if (c.ntt_chunk < 1 || c.ntt_chunk > 4096) c.ntt_chunk = 640;
    c.ntt_unit = unit ? atoi(unit) : 4;
    if (c.ntt_unit < 1 || c.ntt_unit > 255) c.ntt_unit = 4;
  }
  CFHE_CUDA(cudaMalloc(&c.d_error_flag, sizeof(int)));
  CFHE_CUDA(cudaMemset(c.d_error_flag, 0, sizeof(int)));
  c.nqinv.resize(c.NP);
  for (int g = 0; g < c.NP; g++) {
    uint32_t q = c.q[g], x = q;
    for (int i = 0; i < 5; i++) x *= 2u - q * x;  // q^-1 mod 2^32
    c.nqinv[g] = 0u - x;
  }
  const int max_level = (int)c.level_config.size() - 1;
  c.levels.resize(max_level + 2);
  for (int level = -1; level <= max_level; level++) {
    LevelPlan &lp = c.levels[level + 1];
    lp.level = level;
    if (level == -1) {
      lp.num_main = c.level_config[0].first - c.add_main;
      lp.num_ter = c.level_config[0].second - c.add_ter;
      lp.alpha = lp.num_main + lp.num_ter;
      lp.beta = 1;
    } else {
      lp.num_main = c.level_config[level].first;
      lp.num_ter = c.level_config[level].second;
      lp.alpha = c.A;
      lp.beta = (lp.num_main + c.T + c.A - 1) / c.A;
    }
    if (lp.num_main < 0 || lp.num_ter < 0 || lp.alpha > c.A ||
        lp.num_main > c.M || lp.num_ter > c.T) {
      set_error("invalid level table");
      return -1;
    }
    lp.nq = lp.num_main + lp.num_ter;
    lp.ntot = lp.nq + lp.alpha;
    np_limbs(c, lp.num_main, lp.num_ter, 0, lp.q_g);
    np_limbs(c, lp.num_main, lp.num_ter, lp.alpha, lp.full_g);
    if (lp.nq == 0 || lp.alpha == 0) continue;  // nothing to switch
    // digits are alpha-sized windows of the index padded with the absent
    // terminal slots (reference src/core/ModSwitch.cu:204-227)
    const int off = level == -1 ? 0 : c.T - lp.num_ter;
    const int padded = lp.nq + off;
    lp.own_digit.assign(lp.nq, 255);
    for (int i = 0; i < lp.beta; i++) {
      int s0 = i * lp.alpha, s1 = std::min((i + 1) * lp.alpha, padded);
      if (s1 <= off) continue;
      s0 = std::max(0, s0 - off);
      s1 -= off;
      DigitPlan d;
      d.index = i;
      d.s0 = s0;
      d.s1 = s1;
      for (int k = s0; k < s1; k++) {
        d.conv.src_g.push_back(lp.q_g[k]);
        d.conv.src_pos.push_back(k);
        lp.own_digit[k] = (int)lp.digits.size();
      }
      for (int k = 0; k < lp.ntot; k++)
        if (k < s0 || k >= s1) {
          d.conv.dst_g.push_back(lp.full_g[k]);
          d.dst_pos.push_back(k);
        }
      if (int r = finish_conv(c, d.conv, {})) return r;
      lp.digits.push_back(std::move(d));
    }
    std::vector<int> aux(lp.full_g.begin() + lp.nq, lp.full_g.end());
    for (int g : lp.q_g) {
      const uint32_t q = c.q[g];
      lp.p_mont.push_back(to_mont(prod_mod(c, aux, q), q));
    }
    if (int r = build_down(c, lp.down[0], lp.full_g, lp.q_g)) return r;
    if (level >= 1) {
      const LevelPlan &lo = c.levels[level];  // level - 1, built before
      if (int r = build_down(c, lp.down[1], lp.q_g, lo.q_g)) return r;
      if (int r = build_down(c, lp.down[2], lp.full_g, lo.q_g)) return r;
      lp.has_rescale = true;
    }
  }
  return 0;
}

void free_plans(Context &c) {
  for (LevelPlan &lp : c.levels) {
    for (DigitPlan &d : lp.digits)
      {
        if (d.conv.d_table) cudaFree(d.conv.d_table);
        if (d.conv.d_tc_table) cudaFree(d.conv.d_tc_table);
      }
    for (ConvPlan &cv : lp.down) {
      if (cv.d_table) cudaFree(cv.d_table);
      if (cv.d_tc_table) cudaFree(cv.d_tc_table);
    }
  }
  c.levels.clear();
  for (cudaEvent_t e : c.prof_events) cudaEventDestroy(e);
  c.prof_events.clear();
  if (c.ws) cudaFree(c.ws);
  c.ws = nullptr;
  c.ws_words = 0;
  if (c.d_error_flag) cudaFree(c.d_error_flag);
  c.d_error_flag = nullptr;
  if (c.order_event) cudaEventDestroy(c.order_event);
  c.order_event = nullptr;
}

void Context::mark(const char *stage) const {
  if (!profiling) return;
  if (prof_used == prof_events.size()) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    prof_events.push_back(e);
    prof_names.push_back(stage);
  }
  prof_names[prof_used] = stage;
  cudaEventRecord(prof_events[prof_used++], stream);
}

int ensure_workspace(Context &c, size_t words) {
  if (words <= c.ws_words) return 0;
  CFHE_CUDA(cudaStreamSynchronize(c.stream));
  if (c.ws) CFHE_CUDA(cudaFree(c.ws));
  c.ws = nullptr;
  c.ws_words = 0;
  CFHE_CUDA(cudaMalloc(&c.ws, words * sizeof(uint32_t)));
  c.ws_words = words;
  return 0;
}

}  // namespace cfhe
