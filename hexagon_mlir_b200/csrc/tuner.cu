// GEMM dispatch and the per-shape variant search.
//
// The reference searches power-of-two (BM,BN,BK) tiles for its matrix engine
// (qcom_hexagon_backend/backend/hmx_search.py): enumerate, refuse illegal
// candidates with a reason, order by a modelled lower bound, measure each
// (three repetitions, inf on any failure or failed verification), and let a
// challenger take the crown from the incumbent only when it is faster by more
// than max(3 x CV, 15%), the round being void when a canary measurement
// drifted.  Here the candidates are the fixed list of hand-written tensor-core
// variants; the five stages and the gate are the same, and the verdict logic
// is a pure function of the measurements so that it can be driven with
// scripted timings (the reference tests its loop with a fake launcher the same
// way: qcom_hexagon_backend/test/test_hmx_search_loop_contract.py:134-158).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "common.h"

namespace b200 {
namespace {

constexpr double kCvFactor = 3.0;       // hmx_search.py:1184
constexpr double kMarginFloor = 0.15;   // hmx_search.py:1185
constexpr int kReps = 3;                // hexagon_bench reps
constexpr int kSimtVariant = -1;
constexpr double kStreamKFixup = 4000.0;  // clocks to combine one more contributor's partial of a cut tile
constexpr double kStreamKDrift = 0.25;    // modelled loss of the k-block phase, in tile times

std::mutex g_cache_mu;
struct CacheEntry {
  int variant;
  double q50_us;
};
std::map<std::string, CacheEntry> g_cache;

std::string build_fingerprint() {
  std::ostringstream os;
  os << __DATE__ << " " << __TIME__ << " v" << tc_variant_count();
  for (int v = 0; v < tc_variant_count(); ++v) os << ":" << tc_variant_info(v).name;
  return os.str();
}

// Cache identity: shape, dtype/epilogue, device, build (tuning_key_int,
// hmx_search.py:416-443, rotates on the build fingerprint too).
std::string cache_key(int64_t m, int64_t n, int64_t k, int epi) {
  std::ostringstream os;
  os << "f16|" << m << "|" << n << "|" << k << "|e" << epi << "|" << ctx().gpu_name << "|"
     << build_fingerprint();
  return os.str();
}

// Modelled time in SM clocks.  A tile of bm x bn needs bm*bn*64*2 / (8192 * cta_group)
// tensor clocks per 64-deep K block at full rate, and each tiling sustains only a
// measured fraction of that rate (narrow tiles are bound by shared-memory and L2
// traffic per flop); tiles run in waves over the SMs (SM pairs for cta_group 2).
// Orders candidates; never crowns one.
double model_clocks(const TcVariantInfo &vi, int64_t m, int64_t n, int64_t k, int sms) {
  const double tiles = std::ceil((double)m / vi.bm) * std::ceil((double)n / vi.bn);
  const double slots = std::max(1, sms / vi.cta_group);
  const double kblocks = std::ceil((double)k / vi.bk);
  const double per_block = (double)vi.bm * vi.bn * vi.bk * 2.0 / (8192.0 * vi.cta_group) / vi.model_eff;
  if (vi.stream_k) {
    // whole tiles for all rounds but the last full one, then the k-blocks of the last P..2P-1
    // tiles (all tiles below P) dealt out evenly: no round is left part-filled, but the pair that
    // combines a cut tile pulls every other contributor's fp32 partial through the workspace
    if (std::fmod(tiles, slots) == 0.0) return (tiles / slots) * (kblocks * per_block + 1500.0) + 1.0;  // nothing to cut
    const double rem = std::fmod(tiles, slots);
    const double dp_rounds = tiles >= slots ? std::floor(tiles / slots) - (2.0 * rem >= slots ? 0.0 : 1.0) : 0.0;
    const double sk_tiles = tiles - dp_rounds * slots, units = sk_tiles * kblocks;
    const double pairs = std::min(slots, units), share = std::ceil(units / pairs);
    const double others = std::max(1.0, std::ceil(kblocks / share));  // contributors beside the combining pair
    // measured: pairs that run the same tile's k-range out of step share less in L2 than pairs
    // that start their tiles together; charged as a quarter of a tile's time
    return dp_rounds * (kblocks * per_block + 1500.0) + (share + kStreamKDrift * kblocks) * per_block + 1500.0 +
           kStreamKFixup * others;
  }
  const double waves = std::ceil(tiles / slots);
  return waves * (kblocks * per_block + 1500.0);
}

struct Measured {
  int variant;
  std::string label;
  std::string verdict;  // legality
  double model;
  double q50 = INFINITY, q20 = INFINITY, q80 = INFINITY;
  bool measured() const { return std::isfinite(q50) && q50 > 0; }
  double cv() const {  // quantile_spread_cv: (q80-q20)/q50
    if (!measured() || !std::isfinite(q20) || !std::isfinite(q80)) return 0.0;
    return std::max(0.0, (q80 - q20) / q50);
  }
};

double champion_gate(double cv) {
  if (!std::isfinite(cv)) cv = 0.0;
  return std::max(kCvFactor * std::fabs(cv), kMarginFloor);
}

std::string jnum(double v) {
  if (!std::isfinite(v)) return "null";
  char b[64];
  snprintf(b, sizeof(b), "%.6g", v);
  return b;
}

struct CanaryRecord {
  std::string status;
  bool healthy;
  double q50, cv, reference, delta, gate;
};

// canary_verdict (hmx_search.py:1292-1367)
CanaryRecord canary_verdict(const double *canary, double reference_q50) {
  CanaryRecord r{"ok", true, NAN, 0.0, reference_q50, NAN, NAN};
  if (!canary) {
    r.status = "missing";
    r.healthy = false;
    return r;
  }
  Measured m;
  m.q50 = canary[0];
  m.q20 = canary[1];
  m.q80 = canary[2];
  r.cv = m.cv();
  if (!m.measured()) {
    r.status = "unmeasured";
    r.healthy = false;
    return r;
  }
  r.q50 = m.q50;
  if (!std::isfinite(reference_q50) || reference_q50 <= 0.0) {
    r.status = "reference-established";
    return r;
  }
  r.gate = champion_gate(r.cv);
  r.delta = (m.q50 - reference_q50) / reference_q50;
  if (std::fabs(r.delta) > r.gate) {
    r.status = "drift";
    r.healthy = false;
  }
  return r;
}

// judge_champion_round (hmx_search.py:1370-1571): deterministic walk in
// enumeration order starting from the control arm; strict ">" on the gate.
struct Judgement {
  int champion = kSimtVariant;
  bool have_champion = false;
  bool significant = false;
  bool round_valid = false;
  std::string json;
};

Judgement judge_round(std::vector<Measured> rows, int control_variant, const double *canary,
                      double canary_reference, int iters, int64_t m, int64_t n, int64_t k) {
  Judgement J;
  CanaryRecord cr = canary_verdict(canary, canary_reference);
  J.round_valid = cr.healthy;
  std::vector<const Measured *> measured;
  std::vector<std::string> unmeasured;
  for (auto &r : rows) {
    if (r.measured()) measured.push_back(&r);
    else unmeasured.push_back(r.label);
  }
  const Measured *control = nullptr;
  for (auto *r : measured)
    if (r->variant == control_variant) control = r;
  // A control arm that was nominated but scored inf leaves no arm to judge a
  // win against: no champion.  With no control nominated the walk starts at
  // the first enumerated candidate (hmx_search.py:1467-1487).
  bool control_nominated = false;
  for (auto &r : rows) control_nominated |= r.variant == control_variant;
  const Measured *incumbent =
      control ? control : (control_nominated || measured.empty() ? nullptr : measured[0]);
  std::ostringstream cmp;
  bool first = true;
  int step = 0;
  if (incumbent) {
    for (auto *ch : measured) {
      if (ch == incumbent || ch == control) continue;
      const double cv = std::max(ch->cv(), incumbent->cv());
      const double gate = champion_gate(cv);
      const double delta = (incumbent->q50 - ch->q50) / incumbent->q50;
      const bool takeover = delta > gate;
      if (!first) cmp << ",";
      first = false;
      cmp << "{\"step\":" << step++ << ",\"challenger\":\"" << ch->label << "\",\"incumbent\":\""
          << incumbent->label << "\",\"delta_pct\":" << jnum(100.0 * delta)
          << ",\"cv\":" << jnum(cv) << ",\"gate_pct\":" << jnum(100.0 * gate)
          << ",\"outcome\":\"" << (takeover ? "takeover" : "kept") << "\"}";
      if (takeover) incumbent = ch;
    }
  }
  bool beats = false;
  double beats_delta = 0.0, beats_gate = kMarginFloor;
  if (control && incumbent && incumbent != control) {
    const double cv = std::max(control->cv(), incumbent->cv());
    beats_gate = champion_gate(cv);
    beats_delta = (control->q50 - incumbent->q50) / control->q50;
    beats = beats_delta > beats_gate;
  }
  J.have_champion = incumbent != nullptr;
  J.champion = incumbent ? incumbent->variant : kSimtVariant;
  J.significant = J.round_valid && control && beats;

  std::ostringstream os;
  os << "{\"kind\":\"b200-gemm-search-champion\",\"shape_mnk\":[" << m << "," << n << "," << k
     << "],\"round_verdict\":\"" << (J.round_valid ? "valid" : "invalid-canary")
     << "\",\"iters\":" << iters
     << ",\"gate\":{\"form\":\"max(3xCV, 15%)\",\"cv_factor\":" << kCvFactor
     << ",\"margin_floor\":" << kMarginFloor << "}"
     << ",\"canary\":{\"status\":\"" << cr.status << "\",\"healthy\":" << (cr.healthy ? "true" : "false")
     << ",\"q50_us\":" << jnum(cr.q50) << ",\"cv\":" << jnum(cr.cv)
     << ",\"reference_q50_us\":" << jnum(cr.reference) << ",\"delta_pct\":" << jnum(100.0 * cr.delta)
     << ",\"gate_pct\":" << jnum(100.0 * cr.gate) << "}"
     << ",\"measured_configs\":" << measured.size() << ",\"champion\":";
  if (incumbent) os << "\"" << incumbent->label << "\""; else os << "null";
  os << ",\"champion_variant\":" << J.champion
     << ",\"champion_q50_us\":" << jnum(incumbent ? incumbent->q50 : NAN) << ",\"control\":";
  if (control) os << "\"" << control->label << "\""; else os << "null";
  os << ",\"beats_control\":{\"delta_pct\":" << jnum(100.0 * beats_delta)
     << ",\"gate_pct\":" << jnum(100.0 * beats_gate) << ",\"significant\":" << (J.significant ? "true" : "false")
     << "},\"champion_significant\":" << (J.significant ? "true" : "false")
     << ",\"comparisons\":[" << cmp.str() << "],\"unmeasured\":[";
  for (size_t i = 0; i < unmeasured.size(); ++i) os << (i ? "," : "") << "\"" << unmeasured[i] << "\"";
  os << "],\"candidates\":[";
  for (size_t i = 0; i < rows.size(); ++i) {
    const Measured &r = rows[i];
    os << (i ? "," : "") << "{\"cfg\":\"" << r.label << "\",\"variant\":" << r.variant
       << ",\"verdict\":\"" << r.verdict << "\",\"model_clocks\":" << jnum(r.model)
       << ",\"q50_us\":" << jnum(r.q50) << ",\"q20_us\":" << jnum(r.q20)
       << ",\"q80_us\":" << jnum(r.q80) << ",\"cv\":" << jnum(r.cv()) << "}";
  }
  os << "]}";
  J.json = os.str();
  return J;
}

// Candidates in the deterministic visiting order: legal ones by modelled lower
// bound (rank_tile_candidates, hmx_search.py:1030-1067), ties by index.
std::vector<Measured> enumerate(const GemmArgs &g) {
  std::vector<Measured> rows;
  for (int v = 0; v < tc_variant_count(); ++v) {
    Measured r;
    r.variant = v;
    r.label = tc_variant_info(v).name;
    r.verdict = tc_variant_verdict(v, g);
    // (the SwiGLU read-out multiplies by [Wg | Wu] side by side: twice the columns of work per output column)
    r.model = model_clocks(tc_variant_info(v), g.m, g.epilogue == EPI_SWIGLU ? 2 * g.n : g.n, g.k,
                           ctx().sm_count ? ctx().sm_count : 148);
    rows.push_back(r);
  }
  std::stable_sort(rows.begin(), rows.end(), [](const Measured &a, const Measured &b) {
    bool la = a.verdict == "ok", lb = b.verdict == "ok";
    if (la != lb) return la;
    return a.model < b.model;
  });
  return rows;
}

int copy_out(const std::string &s, char *buf, int cap) {
  if (!buf || cap <= 0) return 0;
  size_t n = std::min((size_t)cap - 1, s.size());
  memcpy(buf, s.data(), n);
  buf[n] = 0;
  return (int)s.size();
}

double quantile(std::vector<double> v, double q) {
  if (v.empty()) return INFINITY;
  std::sort(v.begin(), v.end());
  if (v.size() == 1) return v[0];
  double pos = (v.size() - 1) * q;
  size_t lo = (size_t)pos, hi = std::min(lo + 1, v.size() - 1);
  double f = pos - lo;
  return v[lo] * (1 - f) + v[hi] * f;
}

// ---- device-side helpers of the search ------------------------------------------------
// Inputs are multiples of 1/8 in [-1, 1]: every product and every partial sum
// is exact in fp32 for K up to 2^18, so all variants and the CUDA-core
// reference produce identical bits and verification is an equality test.
__global__ void fill_eighths(__half *p, int64_t n, uint32_t seed) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    uint32_t x = (uint32_t)i * 2654435761u + seed;
    x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
    p[i] = __float2half_rn((float)((int)(x % 17u) - 8) * 0.125f);
  }
}
__global__ void count_mismatch(const uint16_t *a, const uint16_t *b, int64_t n, int *out) {
  int bad = 0;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
    bad += a[i] != b[i];
  if (bad) atomicAdd(out, bad);
}

// calibration_iters (hmx_search.py:1159-1171): time-box one measured launch.
int calibration_iters(double per_iter_us, double target_us = 100000.0, int lo = 5, int hi = 1000) {
  double p = std::max(per_iter_us, 1.0);
  return std::max(lo, std::min(hi, (int)(target_us / p)));
}

// One candidate: a discarded launch, then `reps` timed runs of `iters`
// launches; any failure or failed verification scores inf (hexagon_bench,
// hmx_search.py:1109-1156).  Verification runs on the first repetition.
void measure_variant(Measured &row, const GemmArgs &g, const uint16_t *expect, int *d_bad,
                     int *iters_used) {
  if (row.verdict != "ok") return;
  Context &c = ctx();
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return;
  auto once = [&]() { return launch_gemm_tc(row.variant, g); };
  std::vector<double> samples;
  bool ok = once() == 0 && cudaStreamSynchronize(c.stream) == cudaSuccess;
  if (ok && b200mlir_device_status() != 0) ok = false;
  if (ok) {  // verify
    cudaMemsetAsync(d_bad, 0, sizeof(int), c.stream);
    count_mismatch<<<c.sm_count * 4, 256, 0, c.stream>>>((const uint16_t *)g.c, expect, g.m * g.n, d_bad);
    int bad = -1;
    if (cudaMemcpyAsync(&bad, d_bad, sizeof(int), cudaMemcpyDeviceToHost, c.stream) != cudaSuccess ||
        cudaStreamSynchronize(c.stream) != cudaSuccess || bad != 0)
      ok = false;
  }
  int iters = 5;
  if (ok) {  // pilot to size the time box
    cudaEventRecord(e0, c.stream);
    for (int i = 0; i < 3 && ok; ++i) ok = once() == 0;
    cudaEventRecord(e1, c.stream);
    float ms = 0;
    if (ok && cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess)
      iters = calibration_iters(ms * 1000.0 / 3.0);
    else
      ok = false;
  }
  for (int rep = 0; ok && rep < kReps; ++rep) {
    cudaEventRecord(e0, c.stream);
    for (int i = 0; i < iters && ok; ++i) ok = once() == 0;
    cudaEventRecord(e1, c.stream);
    float ms = 0;
    if (ok && cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess)
      samples.push_back(ms * 1000.0 / iters);
    else
      ok = false;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!ok) {
    cudaGetLastError();
    return;
  }
  row.q50 = quantile(samples, 0.5);
  row.q20 = quantile(samples, 0.2);
  row.q80 = quantile(samples, 0.8);
  if (iters_used) *iters_used = iters;
}

double g_canary_reference = NAN;  // previous round's canary median on this device

}  // namespace

// ---- dispatch ----------------------------------------------------------------------------
int choose_gemm_variant(const GemmArgs &g, std::string *why) {
  const int forced = (int)ctx().opt.gemm_variant;
  if (forced >= 0 && forced < tc_variant_count()) {
    const char *v = tc_variant_verdict(forced, g);
    if (!strcmp(v, "ok")) {
      if (why) *why = "option gemmVariant";
      return forced;
    }
    if (why) *why = std::string("forced variant refused: ") + v;
    return kSimtVariant;
  }
  if (forced == 99) {
    if (why) *why = "option gemmVariant=99 (CUDA-core path)";
    return kSimtVariant;
  }
  {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    auto it = g_cache.find(cache_key(g.m, g.n, g.k, g.epilogue));
    if (it != g_cache.end() && it->second.variant >= 0 && it->second.variant < tc_variant_count() &&
        !strcmp(tc_variant_verdict(it->second.variant, g), "ok")) {
      if (why) *why = "autotune cache";
      return it->second.variant;
    }
  }
  std::vector<Measured> rows = enumerate(g);
  if (!rows.empty() && rows[0].verdict == "ok") {
    if (why) *why = "modelled lower bound";
    return rows[0].variant;
  }
  if (why) *why = rows.empty() ? "no variants" : rows[0].verdict;
  return kSimtVariant;
}

int gemm_dispatch(const GemmArgs &g) {
  B200_TRY(ensure_ready());
  if (g.m <= 0 || g.n <= 0) return 0;
  std::string why;
  int v = choose_gemm_variant(g, &why);
  manifest_record(g, v, why);
  if (v >= 0) return launch_gemm_tc(v, g);
  return launch_gemm_simt(g);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200mlir_gemm_variant_count(void) { return tc_variant_count(); }

int b200mlir_gemm_variant_info(int v, char *json, int cap) {
  clear_error();
  if (v < 0 || v >= tc_variant_count())
    return set_error(B200MLIR_ERR_BAD_ARG, "no such gemm variant %d", v);
  const TcVariantInfo &i = tc_variant_info(v);
  std::ostringstream os;
  os << "{\"variant\":" << v << ",\"name\":\"" << i.name << "\",\"tiles\":[" << i.bm << "," << i.bn
     << "," << i.bk << "],\"stages\":" << i.stages << ",\"cta_group\":" << i.cta_group
     << ",\"smem_bytes\":" << i.smem_bytes << ",\"tmem_cols\":" << i.tmem_cols << "}";
  copy_out(os.str(), json, cap);
  return 0;
}

static GemmArgs shape_only(int64_t m, int64_t n, int64_t k) {
  GemmArgs g;
  g.m = m;
  g.n = n;
  g.k = k;
  g.lda = k;
  g.ldb = n;
  g.ldc = n;
  // aligned placeholders: only the legality predicate looks at them
  g.a = g.b = (const void *)(uintptr_t)256;
  g.c = (void *)(uintptr_t)256;
  return g;
}

int b200mlir_gemm_variant_verdict(int v, int64_t m, int64_t n, int64_t k, char *reason, int cap) {
  clear_error();
  if (v < 0 || v >= tc_variant_count()) return -1;
  const char *r = tc_variant_verdict(v, shape_only(m, n, k));
  copy_out(r, reason, cap);
  return !strcmp(r, "ok") ? 1 : 0;
}

int b200mlir_gemm_explain(int64_t m, int64_t n, int64_t k, char *json, int cap) {
  clear_error();
  GemmArgs g = shape_only(m, n, k);
  std::string why;
  int v = choose_gemm_variant(g, &why);
  std::ostringstream os;
  // plan vocabulary of the reference's manifest: "hmx" = engine path taken,
  // "hvx" = vector fallback (HmxManifest.h:81-100)
  os << "{\"shape_mnk\":[" << m << "," << n << "," << k << "],\"plan\":\""
     << (v >= 0 ? "tcgen05" : "cuda-core") << "\",\"reference_plan\":\"" << (v >= 0 ? "hmx" : "hvx")
     << "\",\"variant\":" << v << ",\"name\":\"" << (v >= 0 ? tc_variant_info(v).name : "simt64x64")
     << "\",\"reason\":\"" << why << "\",\"candidates\":[";
  std::vector<Measured> rows = enumerate(g);
  for (size_t i = 0; i < rows.size(); ++i)
    os << (i ? "," : "") << "{\"cfg\":\"" << rows[i].label << "\",\"verdict\":\"" << rows[i].verdict
       << "\",\"model_clocks\":" << jnum(rows[i].model) << "}";
  os << "]}";
  copy_out(os.str(), json, cap);
  return v;
}

// Verdict logic with caller-supplied measurements: times_us[3*v + {0,1,2}] =
// {q50, q20, q80} of variant v (non-finite or <= 0 q50: the candidate failed);
// canary = {q50, q20, q80} or NULL; canary_reference_q50 <= 0 or NaN: none yet.
int b200mlir_gemm_search_scripted(int64_t m, int64_t n, int64_t k, const double *times_us,
                                           int n_variants, int control_variant,
                                           const double *canary, double canary_reference_q50,
                                           char *json, int cap) {
  clear_error();
  if (!times_us || n_variants != tc_variant_count()) {
    set_error(B200MLIR_ERR_BAD_ARG, "scripted search: need %d timing triples", tc_variant_count());
    return -1;
  }
  std::vector<Measured> rows = enumerate(shape_only(m, n, k));
  for (auto &r : rows) {
    if (r.verdict != "ok") continue;
    r.q50 = times_us[3 * r.variant];
    r.q20 = times_us[3 * r.variant + 1];
    r.q80 = times_us[3 * r.variant + 2];
  }
  Judgement J = judge_round(rows, control_variant, canary, canary_reference_q50, 0, m, n, k);
  copy_out(J.json, json, cap);
  if (J.have_champion && J.round_valid) {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    g_cache[cache_key(m, n, k, EPI_F16)] = CacheEntry{J.champion, times_us[3 * J.champion]};
  }
  return J.have_champion ? J.champion : -1;
}

int b200mlir_gemm_autotune(int64_t m, int64_t n, int64_t k, char *json, int cap) {
  clear_error();
  if (ensure_ready()) return -1;
  if (m <= 0 || n <= 0 || k <= 0) {
    set_error(B200MLIR_ERR_BAD_ARG, "autotune: empty shape");
    return -1;
  }
  Context &c = ctx();
  {
    std::lock_guard<std::mutex> lk(g_cache_mu);
    auto it = g_cache.find(cache_key(m, n, k, EPI_F16));
    if (it != g_cache.end()) {
      std::ostringstream os;
      os << "{\"kind\":\"b200-gemm-search-champion\",\"cache_hit\":true,\"champion_variant\":"
         << it->second.variant << ",\"champion_q50_us\":" << jnum(it->second.q50_us) << "}";
      copy_out(os.str(), json, cap);
      return it->second.variant;
    }
  }
  __half *A = nullptr, *B = nullptr, *C = nullptr, *E = nullptr;
  int *d_bad = nullptr;
  auto cleanup = [&]() {
    cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(E); cudaFree(d_bad);
  };
  if (cudaMalloc(&A, (size_t)m * k * 2) != cudaSuccess || cudaMalloc(&B, (size_t)k * n * 2) != cudaSuccess ||
      cudaMalloc(&C, (size_t)m * n * 2) != cudaSuccess || cudaMalloc(&E, (size_t)m * n * 2) != cudaSuccess ||
      cudaMalloc(&d_bad, sizeof(int)) != cudaSuccess) {
    set_error(B200MLIR_ERR_CUDA, "autotune: allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
    cleanup();
    return -1;
  }
  fill_eighths<<<c.sm_count * 8, 256, 0, c.stream>>>(A, m * k, 0x1234u);
  fill_eighths<<<c.sm_count * 8, 256, 0, c.stream>>>(B, k * n, 0x9876u);
  GemmArgs g;
  g.a = A; g.b = B; g.c = E; g.m = m; g.n = n; g.k = k; g.lda = k; g.ldb = n; g.ldc = n;
  if (launch_gemm_simt(g) != 0 || cudaStreamSynchronize(c.stream) != cudaSuccess) {
    cleanup();
    return -1;
  }
  g.c = C;
  // canary first: the smallest variant on a small fixed cube, same protocol
  GemmArgs cg = g;
  cg.m = cg.n = cg.k = std::min<int64_t>(256, std::min(m, std::min(n, k)) / 8 * 8);
  cg.lda = k; cg.ldb = n; cg.ldc = n;
  double canary[3] = {INFINITY, INFINITY, INFINITY};
  bool have_canary = false;
  if (cg.m >= 8) {
    Measured cm;
    cm.variant = tc_variant_count() - 1;
    cm.verdict = tc_variant_verdict(cm.variant, cg);
    // expected values for the canary sub-problem are the top-left block of E only when ld matches; verify by its own reference
    __half *CE = nullptr;
    if (cm.verdict == "ok" && cudaMalloc(&CE, (size_t)m * n * 2) == cudaSuccess) {
      GemmArgs ce = cg; ce.c = CE;
      cudaMemsetAsync(CE, 0, (size_t)m * n * 2, c.stream);
      cudaMemsetAsync(C, 0, (size_t)m * n * 2, c.stream);
      if (launch_gemm_simt(ce) == 0) {
        measure_variant(cm, cg, (const uint16_t *)CE, d_bad, nullptr);
        canary[0] = cm.q50; canary[1] = cm.q20; canary[2] = cm.q80;
        have_canary = true;
      }
      cudaStreamSynchronize(c.stream);
      cudaFree(CE);
    }
  }
  std::vector<Measured> rows = enumerate(g);
  int iters = 0;
  for (auto &r : rows) measure_variant(r, g, (const uint16_t *)E, d_bad, &iters);
  int control = rows.empty() ? -1 : rows[0].variant;  // the dispatcher's own pick defends the crown
  Judgement J = judge_round(rows, control, have_canary ? canary : nullptr, g_canary_reference, iters, m, n, k);
  if (have_canary && std::isfinite(canary[0]) && (J.round_valid)) g_canary_reference = canary[0];
  copy_out(J.json, json, cap);
  if (J.have_champion && J.round_valid) {
    double q = INFINITY;
    for (auto &r : rows) if (r.variant == J.champion) q = r.q50;
    std::lock_guard<std::mutex> lk(g_cache_mu);
    g_cache[cache_key(m, n, k, EPI_F16)] = CacheEntry{J.champion, q};
  }
  cleanup();
  clear_error();
  return J.have_champion ? J.champion : -1;
}

int b200mlir_autotune_cache_save(const char *path) {
  clear_error();
  if (!path) return set_error(B200MLIR_ERR_BAD_ARG, "cache_save: null path");
  std::lock_guard<std::mutex> lk(g_cache_mu);
  std::ofstream f(path);
  if (!f) return set_error(B200MLIR_ERR_BAD_ARG, "cache_save: cannot open %s", path);
  f << "{\"kind\":\"b200-gemm-autotune-cache\",\"entries\":[\n";
  bool first = true;
  for (auto &kv : g_cache) {
    f << (first ? "" : ",\n") << "{\"key\":\"" << kv.first << "\",\"variant\":" << kv.second.variant
      << ",\"q50_us\":" << jnum(kv.second.q50_us) << "}";
    first = false;
  }
  f << "\n]}\n";
  return 0;
}

int b200mlir_autotune_cache_load(const char *path) {
  clear_error();
  if (!path) return set_error(B200MLIR_ERR_BAD_ARG, "cache_load: null path");
  std::ifstream f(path);
  if (!f) return set_error(B200MLIR_ERR_BAD_ARG, "cache_load: cannot open %s", path);
  std::string line;
  int loaded = 0;
  std::lock_guard<std::mutex> lk(g_cache_mu);
  while (std::getline(f, line)) {
    size_t kp = line.find("\"key\":\"");
    size_t vp = line.find("\"variant\":");
    if (kp == std::string::npos || vp == std::string::npos) continue;
    kp += 7;
    size_t ke = line.find('"', kp);
    if (ke == std::string::npos) continue;
    CacheEntry e;
    e.variant = atoi(line.c_str() + vp + 10);
    e.q50_us = NAN;
    size_t qp = line.find("\"q50_us\":");
    if (qp != std::string::npos) e.q50_us = atof(line.c_str() + qp + 9);
    g_cache[line.substr(kp, ke - kp)] = e;  // entries from another build/device never match a key
    ++loaded;
  }
  return loaded >= 0 ? 0 : 0;
}

void b200mlir_autotune_cache_clear(void) {
  std::lock_guard<std::mutex> lk(g_cache_mu);
  g_cache.clear();
}

}  // extern "C"
