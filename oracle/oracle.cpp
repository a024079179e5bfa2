// TEST INFRASTRUCTURE — CPU oracle for the hybrid DeltaNet / attention / MoE token loop.
// Not product code. See oracle.h for what is and is not pinned by reference fixtures.
//
// Each function cites the reference file:line it restates. Arithmetic follows the
// reference's CPU code: serial f32 dot products, f64 sums inside the norms, f64
// transcendental functions narrowed to f32.
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "oracle_quant.h"

using namespace orc;

namespace {

struct Tensor {
  uint32_t type = 0;
  int64_t ne[4] = {1, 1, 1, 1};
  const uint8_t* data = nullptr;
  int64_t rb = 0;  // bytes per row
  bool ok() const { return data != nullptr; }
  const uint8_t* row(int64_t r) const { return data + r * rb; }
};

struct Layer {
  bool is_attn = false;
  Tensor attn_norm, ffn_norm;
  // DeltaNet (llm/deltanet.go:134-154)
  Tensor qkv, z, alpha, beta, conv1d, ssm_a, dt_bias, ssm_norm, ssm_out;
  // attention (llm/attn.go:76-93)
  Tensor q, k, v, o, q_norm, k_norm;
  // MoE (llm/moe.go:115-123)
  Tensor router, sh_gate_inp, gate_exps, up_exps, down_exps, gate_sh, up_sh, down_sh;
  // draft extras (llm/mtp.go:36-48)
  Tensor enorm, hnorm, eh_proj, head_norm;
};

inline bool dev_like(int numerics) { return (numerics & 0xff) == ORC_DEVICE_LIKE; }
inline bool w16(int numerics, int bit) { return (numerics & bit) != 0; }
inline float sigmoidf_(float x) { return (float)(1.0 / (1.0 + std::exp(-(double)x))); }  // llm/hc.go:266
inline float siluf_(float x) { return x * sigmoidf_(x); }                                // llm/hc.go:268

// llm/deltanet.go:445-455: float32 add inside the log, identity above 20.
inline float softplusf_(float x) {
  if (x > 20) return x;
  float e = (float)std::exp((double)x);
  float s = 1.0f + e;
  return (float)std::log((double)s);
}

std::vector<float> to_f32(const Tensor& t) {
  int64_t n = t.ne[0] * t.ne[1] * t.ne[2] * t.ne[3];
  std::vector<float> v((size_t)n);
  dequantize(t.type, t.data, n, v.data());
  return v;
}

// y = W x over rows [0, rows) of t starting at row0; serial f32 sum (llm/hc.go:255-264).
// w16: every weight is an fp16 value, as in the reference's many-row tensor-core GEMMs, which round the
// dequantised weight when they unpack a slab into LDS (shaders/llm_gemm.comp MODE 2,
// shaders/llm_moe_gemm.comp:260-261, 428-430; formed as dequantize_w16 describes); its decode GEMVs keep
// the f32 value.
void matvec(const Tensor& t, int64_t row0, int64_t rows, const float* x, float* y, bool w16 = false) {
  const int64_t k = t.ne[0];
#pragma omp parallel
  {
    std::vector<float> buf((size_t)k);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
      const float* w;
      if (t.type == T_F32) {
        w = (const float*)t.row(row0 + r);
      } else {
        if (w16) dequantize_w16(t.type, t.row(row0 + r), k, buf.data());
        else dequantize(t.type, t.row(row0 + r), k, buf.data());
        w = buf.data();
      }
      float s = 0;
      for (int64_t i = 0; i < k; i++) s += w[i] * x[i];
      y[r] = s;
    }
  }
}

void rmsnorm(const float* src, const float* gamma, int n, float eps, float* dst) {
  double ss = 0;
  for (int i = 0; i < n; i++) ss += (double)src[i] * (double)src[i];
  float scale = (float)(1.0 / std::sqrt(ss / (double)n + (double)eps));
  for (int i = 0; i < n; i++) dst[i] = src[i] * scale * gamma[i];
}

void round_f16(float* x, int64_t n) { for (int64_t i = 0; i < n; i++) x[i] = f16_round(x[i]); }

}  // namespace

struct orc_model {
  orc_config c;
  std::vector<Layer> layers;  // n_layer (+1 draft)
  Tensor token_embd, output, output_norm;
  // small f32 tensors pre-dequantised
  struct Small {
    std::vector<float> attn_norm, ffn_norm, conv1d, ssm_a, dt_bias, ssm_norm, q_norm, k_norm, sh_gate_inp, enorm, hnorm, head_norm;
  };
  std::vector<Small> small;
  std::vector<float> out_norm;
};

struct orc_seq {
  const orc_model* m = nullptr;
  int past = 0;
  bool draft = false;
  // per layer
  struct L {
    std::vector<float> K, V;     // attention: [cell][n_kv][hd]
    std::vector<float> conv, S;  // DeltaNet: conv ring [cw][conv-1] (column 0 oldest), S [Hv][d][d] transposed
  };
  std::vector<L> l;
};

namespace {

struct Work {
  std::vector<float> xn, proj, z, ab, conv, qn, kn, o, fin, mix, logits, probs, g, u, sw, down, ffn, sh;
  std::vector<float> q, gate, kk, vv, ctx, scores;
  std::vector<int32_t> idx;
};

// One DeltaNet layer for one token (llm/deltanet.go:212-352, nTok = 1).
void deltanet_token(const orc_model& m, int li, orc_seq::L& st, const float* xn, int numerics, float* out, Work& w) {
  const orc_config& c = m.c;
  const Layer& L = m.layers[li];
  const auto& sm = m.small[li];
  const int d = c.dn_head_dim, Hk = c.dn_heads_k, Hv = c.dn_heads_v, K = c.dn_conv;
  const int qk = Hk * d, vw = Hv * d, cw = 2 * qk + vw, hist = K - 1;
  w.proj.resize(cw); w.z.resize(vw); w.ab.resize(2 * Hv);
  matvec(L.qkv, 0, cw, xn, w.proj.data(), w16(numerics, ORC_W16_DN_QKV));
  matvec(L.z, 0, vw, xn, w.z.data(), w16(numerics, ORC_W16_DN_GATE));
  matvec(L.alpha, 0, Hv, xn, w.ab.data());
  matvec(L.beta, 0, Hv, xn, w.ab.data() + Hv);
  // decay and write strength (llm/deltanet.go:266-271)
  std::vector<float> gate(Hv), beta(Hv);
  for (int h = 0; h < Hv; h++) {
    gate[h] = softplusf_(w.ab[h] + sm.dt_bias[h]) * sm.ssm_a[h];
    beta[h] = sigmoidf_(w.ab[Hv + h]);
  }
  // depthwise causal conv over history + this token, then SiLU (llm/deltanet.go:276-300)
  w.conv.resize(cw);
  for (int ch = 0; ch < cw; ch++) {
    const float* kx = &sm.conv1d[(size_t)ch * K];
    float s = 0;
    for (int j = 0; j < K; j++) {
      int p = j - hist;  // token index; negative reads the history
      float x = p < 0 ? st.conv[(size_t)ch * hist + hist + p] : w.proj[ch];
      s += x * kx[j];
    }
    w.conv[ch] = siluf_(s);
  }
  // new history: the last conv-1 inputs (llm/deltanet.go:305-316)
  for (int ch = 0; ch < cw; ch++) {
    for (int p = 0; p + 1 < hist; p++) st.conv[(size_t)ch * hist + p] = st.conv[(size_t)ch * hist + p + 1];
    st.conv[(size_t)ch * hist + hist - 1] = w.proj[ch];
  }
  // L2 norm of q and k per head, x/sqrt(|x|^2 + eps) (llm/deltanet.go:423-443, L2Rsqrt)
  w.qn.resize(qk); w.kn.resize(qk);
  for (int r = 0; r < 2 * Hk; r++) {
    const float* row = &w.conv[(size_t)r * d];
    double ss = 0;
    for (int i = 0; i < d; i++) ss += (double)row[i] * (double)row[i];
    float scale = (float)(1.0 / std::sqrt(ss + (double)c.eps));
    float* o = r < Hk ? &w.qn[(size_t)r * d] : &w.kn[(size_t)(r - Hk) * d];
    for (int i = 0; i < d; i++) o[i] = row[i] * scale;
  }
  const float* v = &w.conv[2 * qk];
  // gated delta rule (llm/deltanet.go:365-403), V head h reads K head h % Hk (:412-418)
  w.o.resize(vw);
  const float scale = (float)(1.0 / std::sqrt((double)d));
#pragma omp parallel for schedule(static)
  for (int h = 0; h < Hv; h++) {
    int hk = h % Hk;
    float* s = &st.S[(size_t)h * d * d];
    const float* q = &w.qn[(size_t)hk * d];
    const float* k = &w.kn[(size_t)hk * d];
    float g = (float)std::exp((double)gate[h]);
    for (int j = 0; j < d * d; j++) s[j] *= g;
    for (int j = 0; j < d; j++) {
      float* row = s + (size_t)j * d;
      float sum = 0;
      for (int x = 0; x < d; x++) sum += row[x] * k[x];
      float dj = (v[h * d + j] - sum) * beta[h];
      float so = 0;
      for (int x = 0; x < d; x++) {
        row[x] += dj * k[x];
        so += row[x] * q[x];
      }
      w.o[h * d + j] = so * scale;
    }
  }
  // gated RMSNorm per V head x shared gamma x sigmoid(z) (llm/deltanet.go:329-341)
  w.fin.resize(vw);
  for (int h = 0; h < Hv; h++) {
    const float* x = &w.o[(size_t)h * d];
    double ss = 0;
    for (int i = 0; i < d; i++) ss += (double)x[i] * (double)x[i];
    float sc = (float)(1.0 / std::sqrt(ss / (double)d + (double)c.eps));
    for (int j = 0; j < d; j++) w.fin[h * d + j] = x[j] * sc * sm.ssm_norm[j] * sigmoidf_(w.z[h * d + j]);
  }
  if (dev_like(numerics)) round_f16(w.fin.data(), vw);
  matvec(L.ssm_out, 0, c.n_embd, w.fin.data(), out, w16(numerics, ORC_W16_DN_OUT));
}

// NeoX partial rotary on the first rope_dims of each head, angle walked in f64
// (llm/attn.go:554-584 with text positions).
void rope(const orc_config& c, float* x, int n_heads, int pos) {
  int rot = std::min(c.rope_dims, c.head_dim);
  int half = rot / 2;
  double scale = std::pow((double)c.rope_base, -2.0 / (double)rot);
  double theta = (double)pos;
  for (int i = 0; i < half; i++) {
    float cs = (float)std::cos(theta), sn = (float)std::sin(theta);
    for (int h = 0; h < n_heads; h++) {
      float* row = x + (size_t)h * c.head_dim;
      float x0 = row[i], x1 = row[i + half];
      row[i] = x0 * cs - x1 * sn;
      row[i + half] = x0 * sn + x1 * cs;
    }
    theta *= scale;
  }
}

// One gated-GQA attention layer for one token at cell `cell` with rotary position `pos`
// (llm/attn.go:135-219 dense arm, :444-496 attention, :510-522 headNorm).
void attn_token(const orc_model& m, int li, orc_seq::L& st, const float* xn, int cell, int pos, int numerics, float* out, Work& w) {
  const orc_config& c = m.c;
  const Layer& L = m.layers[li];
  const auto& sm = m.small[li];
  const int hd = c.head_dim, H = c.n_head, Hkv = c.n_head_kv, kvw = Hkv * hd;
  std::vector<float> qfull((size_t)H * 2 * hd);
  w.q.resize((size_t)H * hd); w.gate.resize((size_t)H * hd); w.kk.resize(kvw); w.vv.resize(kvw);
  matvec(L.q, 0, (int64_t)H * 2 * hd, xn, qfull.data(), w16(numerics, ORC_W16_ATTN_Q));
  matvec(L.k, 0, kvw, xn, w.kk.data(), w16(numerics, ORC_W16_ATTN_K));
  matvec(L.v, 0, kvw, xn, w.vv.data(), w16(numerics, ORC_W16_ATTN_V));
  for (int h = 0; h < H; h++) {  // per head: hd query rows then hd gate rows (llm/attn.go:162-166)
    memcpy(&w.q[(size_t)h * hd], &qfull[(size_t)h * 2 * hd], sizeof(float) * hd);
    memcpy(&w.gate[(size_t)h * hd], &qfull[(size_t)h * 2 * hd + hd], sizeof(float) * hd);
  }
  for (int h = 0; h < H; h++) rmsnorm(&w.q[(size_t)h * hd], sm.q_norm.data(), hd, c.eps, &w.q[(size_t)h * hd]);
  for (int h = 0; h < Hkv; h++) rmsnorm(&w.kk[(size_t)h * hd], sm.k_norm.data(), hd, c.eps, &w.kk[(size_t)h * hd]);
  rope(c, w.q.data(), H, pos);
  rope(c, w.kk.data(), Hkv, pos);
  if (dev_like(numerics)) {  // fp16 cache and fp16 query (llm/attn.go:176-184, 196-199)
    round_f16(w.kk.data(), kvw); round_f16(w.vv.data(), kvw); round_f16(w.q.data(), (int64_t)H * hd);
  }
  if ((int64_t)st.K.size() < (int64_t)(cell + 1) * kvw) { st.K.resize((size_t)(cell + 1) * kvw); st.V.resize((size_t)(cell + 1) * kvw); }
  memcpy(&st.K[(size_t)cell * kvw], w.kk.data(), sizeof(float) * kvw);
  memcpy(&st.V[(size_t)cell * kvw], w.vv.data(), sizeof(float) * kvw);
  const int rep = H / Hkv, n = cell + 1;
  const float scale = (float)(1.0 / std::sqrt((double)hd));
  w.ctx.assign((size_t)H * hd, 0.f);
#pragma omp parallel
  {
    std::vector<float> scores((size_t)n);
#pragma omp for schedule(static)
    for (int h = 0; h < H; h++) {
      int kvh = h / rep;
      const float* qv = &w.q[(size_t)h * hd];
      for (int j = 0; j < n; j++) {
        const float* kv = &st.K[((size_t)j * Hkv + kvh) * hd];
        float s = 0;
        for (int dd = 0; dd < hd; dd++) s += qv[dd] * kv[dd];
        scores[j] = s * scale;
      }
      float mx = scores[0];
      for (int j = 1; j < n; j++) if (scores[j] > mx) mx = scores[j];
      float sum = 0;
      for (int j = 0; j < n; j++) { scores[j] = (float)std::exp((double)(scores[j] - mx)); sum += scores[j]; }
      float* dst = &w.ctx[(size_t)h * hd];
      if (dev_like(numerics)) {
        // Device-like: probabilities meet the fp16 values as fp16 and the division by
        // the f32 row sum comes last (shaders/llm_attn_wmma.comp:860, llm_attn_combine.comp:70-102).
        for (int j = 0; j < n; j++) {
          float p = f16_round(scores[j]);
          const float* vv = &st.V[((size_t)j * Hkv + kvh) * hd];
          for (int dd = 0; dd < hd; dd++) dst[dd] += p * vv[dd];
        }
        for (int dd = 0; dd < hd; dd++) dst[dd] /= sum;
      } else {
        for (int j = 0; j < n; j++) {
          float wgt = scores[j] / sum;
          const float* vv = &st.V[((size_t)j * Hkv + kvh) * hd];
          for (int dd = 0; dd < hd; dd++) dst[dd] += wgt * vv[dd];
        }
      }
    }
  }
  for (int i = 0; i < H * hd; i++) w.ctx[i] = w.ctx[i] * sigmoidf_(w.gate[i]);  // gate on the output (llm/attn.go:203-208)
  if (dev_like(numerics)) round_f16(w.ctx.data(), (int64_t)H * hd);
  matvec(L.o, 0, c.n_embd, w.ctx.data(), out, w16(numerics, ORC_W16_ATTN_OUT));
}

// Routed + shared MoE block for one token (llm/moe.go:219-409). x is the f32 norm
// output, xr the same vector as the matmuls see it (fp16-rounded when device-like).
void moe_token(const orc_model& m, int li, const float* x, const float* xr, int numerics, float* out,
               int32_t* topk_out, float* topkw_out, float* margin_out, Work& w, const int32_t* forced = nullptr) {
  const orc_config& c = m.c;
  const Layer& L = m.layers[li];
  const auto& sm = m.small[li];
  const int nE = c.n_expert, used = c.n_expert_used, ff = c.ffn_expert, ffs = c.ffn_shared, H = c.n_embd;
  w.logits.resize(nE); w.probs.resize(nE); w.idx.resize(nE);
  matvec(L.router, 0, nE, xr, w.logits.data(), w16(numerics, ORC_W16_ROUTER));
  {  // softmaxInto (llm/moe.go:426-443)
    float mx = -INFINITY;
    for (int e = 0; e < nE; e++) if (w.logits[e] > mx) mx = w.logits[e];
    float sum = 0;
    for (int e = 0; e < nE; e++) { float v = (float)std::exp((double)(w.logits[e] - mx)); w.probs[e] = v; sum += v; }
    float inv = 1 / sum;
    for (int e = 0; e < nE; e++) w.probs[e] *= inv;
  }
  for (int e = 0; e < nE; e++) w.idx[e] = e;
  // descending probability, equal probabilities keep ascending index (llm/moe.go:249-252)
  std::stable_sort(w.idx.begin(), w.idx.end(), [&](int a, int b) { return w.probs[a] > w.probs[b]; });
  if (topk_out) for (int k = 0; k < used; k++) topk_out[k] = w.idx[k];
  if (margin_out) {
    float pk = w.probs[w.idx[used - 1]], pn = used < nE ? w.probs[w.idx[used]] : 0.f;
    *margin_out = pk > 0 ? (pk - pn) / pk : 0.f;
  }
  // a checker may make the block follow another implementation's selection (same weights rule, its experts)
  if (forced != nullptr && forced[0] >= 0) for (int k = 0; k < used; k++) w.idx[k] = forced[k];
  float sum = 0;
  std::vector<float> wt(used);
  for (int k = 0; k < used; k++) { wt[k] = w.probs[w.idx[k]]; sum += wt[k]; }
  if (sum < 6.103515625e-5f) sum = 6.103515625e-5f;  // llm/moe.go:256-282
  for (int k = 0; k < used; k++) wt[k] = wt[k] / sum;
  if (topkw_out) for (int k = 0; k < used; k++) topkw_out[k] = wt[k];
  // routed experts, weights after the FFN, summed in slot order (llm/moe.go:289-359)
  w.g.resize(std::max(ff, ffs)); w.u.resize(std::max(ff, ffs)); w.sw.resize(std::max(ff, ffs)); w.down.resize(H);
  for (int j = 0; j < H; j++) out[j] = 0;
  for (int k = 0; k < used; k++) {
    int e = w.idx[k];
    const bool ew = w16(numerics, ORC_W16_EXPERTS);
    matvec(L.gate_exps, (int64_t)e * ff, ff, xr, w.g.data(), ew);
    matvec(L.up_exps, (int64_t)e * ff, ff, xr, w.u.data(), ew);
    for (int j = 0; j < ff; j++) w.sw[j] = siluf_(w.g[j]) * w.u[j];
    if (dev_like(numerics)) round_f16(w.sw.data(), ff);  // shaders/llm_moe_gemv.comp:777-781
    matvec(L.down_exps, (int64_t)e * H, H, w.sw.data(), w.down.data(), ew);
    for (int j = 0; j < H; j++) out[j] += w.down[j] * wt[k];
  }
  // shared expert and its one-column sigmoid gate (llm/moe.go:363-409). Device-like: the
  // gate column sees the same fp16 vector as the router (llm/gpu_moe.go:27-33).
  const bool sw16 = w16(numerics, ORC_W16_SHARED);
  matvec(L.gate_sh, 0, ffs, xr, w.g.data(), sw16);
  matvec(L.up_sh, 0, ffs, xr, w.u.data(), sw16);
  for (int j = 0; j < ffs; j++) w.sw[j] = siluf_(w.g[j]) * w.u[j];
  if (dev_like(numerics)) round_f16(w.sw.data(), ffs);
  w.sh.resize(H);
  matvec(L.down_sh, 0, H, w.sw.data(), w.sh.data(), sw16);
  const float* gx = dev_like(numerics) ? xr : x;
  float gl = 0;
  for (int j = 0; j < H; j++) gl += sm.sh_gate_inp[j] * gx[j];
  float s = sigmoidf_(gl);
  for (int j = 0; j < H; j++) out[j] = out[j] + w.sh[j] * s;
}

void embed_row(const orc_model& m, int32_t id, float* dst) {  // llm/model.go:125-144
  dequantize(m.token_embd.type, m.token_embd.row(id), m.c.n_embd, dst);
}

// One layer (mixer + MoE) on the residual h for one token.
void layer_token(const orc_model& m, int li, orc_seq::L& st, float* h, int cell, int pos, int numerics, Work& w,
                 float* mix_out, float* ffn_out, int32_t* topk, float* topkw, float* margin, const int32_t* forced = nullptr) {
  const orc_config& c = m.c;
  const int H = c.n_embd;
  const auto& sm = m.small[li];
  w.xn.resize(H); w.mix.resize(H); w.ffn.resize(H);
  rmsnorm(h, sm.attn_norm.data(), H, c.eps, w.xn.data());
  if (dev_like(numerics)) round_f16(w.xn.data(), H);
  if (m.layers[li].is_attn) attn_token(m, li, st, w.xn.data(), cell, pos, numerics, w.mix.data(), w);
  else deltanet_token(m, li, st, w.xn.data(), numerics, w.mix.data(), w);
  if (mix_out) memcpy(mix_out, w.mix.data(), sizeof(float) * H);
  for (int j = 0; j < H; j++) h[j] += w.mix[j];
  std::vector<float> x(H), xr(H);
  rmsnorm(h, sm.ffn_norm.data(), H, c.eps, x.data());
  xr = x;
  if (dev_like(numerics)) round_f16(xr.data(), H);
  moe_token(m, li, x.data(), xr.data(), numerics, w.ffn.data(), topk, topkw, margin, w, forced);
  if (ffn_out) memcpy(ffn_out, w.ffn.data(), sizeof(float) * H);
  for (int j = 0; j < H; j++) h[j] += w.ffn[j];
}

bool find(const std::map<std::string, Tensor>& t, const std::string& n, Tensor* out) {
  auto it = t.find(n);
  if (it == t.end()) return false;
  *out = it->second;
  return true;
}

}  // namespace

extern "C" {

uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
int64_t orc_row_bytes(uint32_t type, int64_t n) { return row_bytes(type, n); }
int orc_dequantize(uint32_t type, const void* data, int64_t n, float* dst) { return dequantize(type, data, n, dst); }
int orc_dequantize_w16(uint32_t type, const void* data, int64_t n, float* dst) { return dequantize_w16(type, data, n, dst); }
int orc_quantize(uint32_t type, const float* src, int64_t rows, int64_t k, void* dst) { return quantize(type, src, rows, k, dst); }

int orc_matvec(uint32_t type, const void* wd, int64_t rows, int64_t k, const float* x, float* y) {
  Tensor t; t.type = type; t.ne[0] = k; t.ne[1] = rows; t.data = (const uint8_t*)wd; t.rb = row_bytes(type, k);
  if (t.rb < 0) return -1;
  matvec(t, 0, rows, x, y);
  return 0;
}

void orc_rmsnorm(const float* src, const float* gamma, int n, float eps, float* dst) { rmsnorm(src, gamma, n, eps, dst); }

int32_t orc_argmax(const float* logits, int64_t n) {  // llm/sample.go:359-367, ties to the lowest id
  int32_t best = 0; float bv = -INFINITY;
  for (int64_t i = 0; i < n; i++) if (logits[i] > bv) { best = (int32_t)i; bv = logits[i]; }
  return best;
}

orc_model* orc_model_create(const orc_config* cfg, const orc_tensor* tensors, int n_tensors, char* err, int err_len) {
  auto fail = [&](const std::string& s) -> orc_model* { if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", s.c_str()); return nullptr; };
  std::map<std::string, Tensor> tm;
  for (int i = 0; i < n_tensors; i++) {
    Tensor t; t.type = tensors[i].type; t.data = (const uint8_t*)tensors[i].data;
    for (uint32_t d = 0; d < tensors[i].n_dims && d < 4; d++) t.ne[d] = tensors[i].dims[d];
    t.rb = row_bytes(t.type, t.ne[0]);
    if (t.rb < 0) return fail(std::string("bad type/row length for ") + tensors[i].name);
    tm[tensors[i].name] = t;
  }
  auto* m = new orc_model();
  m->c = *cfg;
  const orc_config& c = m->c;
  if (!find(tm, "token_embd.weight", &m->token_embd)) { delete m; return fail("token_embd.weight missing"); }
  if (!find(tm, "output.weight", &m->output)) m->output = m->token_embd;
  if (!find(tm, "output_norm.weight", &m->output_norm)) { delete m; return fail("output_norm.weight missing"); }
  m->out_norm = to_f32(m->output_norm);
  int nl = c.n_layer + (c.has_draft ? 1 : 0);
  m->layers.resize(nl); m->small.resize(nl);
  for (int l = 0; l < nl; l++) {
    Layer& L = m->layers[l]; auto& sm = m->small[l];
    std::string p = "blk." + std::to_string(l) + ".";
    std::string missing;
    auto need = [&](const char* n, Tensor* t) { if (!find(tm, p + n + ".weight", t) && !find(tm, p + n, t)) missing += std::string(" ") + n; };
    L.is_attn = tm.count(p + "attn_q.weight") > 0;  // llm/model.go:377, :443
    need("attn_norm", &L.attn_norm); need("ffn_norm", &L.ffn_norm);
    if (L.is_attn) {
      need("attn_q", &L.q); need("attn_k", &L.k); need("attn_v", &L.v); need("attn_output", &L.o);
      need("attn_q_norm", &L.q_norm); need("attn_k_norm", &L.k_norm);
    } else {
      need("attn_qkv", &L.qkv); need("attn_gate", &L.z); need("ssm_alpha", &L.alpha); need("ssm_beta", &L.beta);
      need("ssm_conv1d", &L.conv1d); need("ssm_a", &L.ssm_a); need("ssm_dt.bias", &L.dt_bias); need("ssm_norm", &L.ssm_norm);
      need("ssm_out", &L.ssm_out);
    }
    need("ffn_gate_inp", &L.router); need("ffn_gate_inp_shexp", &L.sh_gate_inp);
    need("ffn_gate_exps", &L.gate_exps); need("ffn_up_exps", &L.up_exps); need("ffn_down_exps", &L.down_exps);
    need("ffn_gate_shexp", &L.gate_sh); need("ffn_up_shexp", &L.up_sh); need("ffn_down_shexp", &L.down_sh);
    if (l == c.n_layer) { need("nextn.enorm", &L.enorm); need("nextn.hnorm", &L.hnorm); need("nextn.eh_proj", &L.eh_proj); need("nextn.shared_head_norm", &L.head_norm); }
    if (!missing.empty()) { delete m; return fail("layer " + std::to_string(l) + " missing:" + missing); }
    sm.attn_norm = to_f32(L.attn_norm); sm.ffn_norm = to_f32(L.ffn_norm); sm.sh_gate_inp = to_f32(L.sh_gate_inp);
    if (L.is_attn) { sm.q_norm = to_f32(L.q_norm); sm.k_norm = to_f32(L.k_norm); }
    else { sm.conv1d = to_f32(L.conv1d); sm.ssm_a = to_f32(L.ssm_a); sm.dt_bias = to_f32(L.dt_bias); sm.ssm_norm = to_f32(L.ssm_norm); }
    if (l == c.n_layer) { sm.enorm = to_f32(L.enorm); sm.hnorm = to_f32(L.hnorm); sm.head_norm = to_f32(L.head_norm); }
  }
  return m;
}

void orc_model_destroy(orc_model* m) { delete m; }

static void seq_init_layer(const orc_model* m, int li, orc_seq::L& l) {
  const orc_config& c = m->c;
  if (!m->layers[li].is_attn) {
    int cw = 2 * c.dn_heads_k * c.dn_head_dim + c.dn_heads_v * c.dn_head_dim;
    l.conv.assign((size_t)cw * (c.dn_conv - 1), 0.f);
    l.S.assign((size_t)c.dn_heads_v * c.dn_head_dim * c.dn_head_dim, 0.f);
  }
}

orc_seq* orc_seq_create(const orc_model* m) {
  auto* s = new orc_seq(); s->m = m; s->l.resize(m->c.n_layer);
  for (int i = 0; i < m->c.n_layer; i++) seq_init_layer(m, i, s->l[i]);
  return s;
}

orc_seq* orc_draft_seq_create(const orc_model* m) {
  if (!m->c.has_draft) return nullptr;
  auto* s = new orc_seq(); s->m = m; s->draft = true; s->l.resize(1);
  seq_init_layer(m, m->c.n_layer, s->l[0]);
  return s;
}

orc_seq* orc_seq_clone(const orc_seq* s) { return new orc_seq(*s); }
void orc_seq_destroy(orc_seq* s) { delete s; }
int32_t orc_seq_past(const orc_seq* s) { return s->past; }

int orc_extend(const orc_model* m, orc_seq* s, const int32_t* ids, int n, int numerics, float* logits_last, const orc_trace* tr) {
  const orc_config& c = m->c;
  const int H = c.n_embd, nl = c.n_layer, used = c.n_expert_used;
  if (s->draft) return -2;
  Work w;
  std::vector<float> h(H), xn(H), logits;
  for (int t = 0; t < n; t++) {
    if (ids[t] < 0 || ids[t] >= c.vocab) return -1;
    embed_row(*m, ids[t], h.data());
    int pos = s->past;
    for (int l = 0; l < nl; l++) {
      size_t o = (size_t)t * nl + l;
      layer_token(*m, l, s->l[l], h.data(), pos, pos, numerics, w,
                  tr && tr->mix_out ? tr->mix_out + o * H : nullptr, tr && tr->ffn_out ? tr->ffn_out + o * H : nullptr,
                  tr && tr->topk ? tr->topk + o * used : nullptr, tr && tr->topk_w ? tr->topk_w + o * used : nullptr,
                  tr && tr->margin ? tr->margin + o : nullptr, tr && tr->force_topk ? tr->force_topk + o * used : nullptr);
      if (tr && tr->hidden) memcpy(tr->hidden + o * H, h.data(), sizeof(float) * H);
    }
    s->past++;
    bool want = (tr && tr->logits) || (logits_last && t == n - 1) || (tr && tr->normed);
    if (!want) continue;
    rmsnorm(h.data(), m->out_norm.data(), H, c.eps, xn.data());
    if (tr && tr->normed) memcpy(tr->normed + (size_t)t * H, xn.data(), sizeof(float) * H);
    if (dev_like(numerics)) round_f16(xn.data(), H);
    if ((tr && tr->logits) || (logits_last && t == n - 1)) {
      logits.resize(c.vocab);
      matvec(m->output, 0, c.vocab, xn.data(), logits.data(), w16(numerics, ORC_W16_HEAD));
      if (tr && tr->logits) memcpy(tr->logits + (size_t)t * c.vocab, logits.data(), sizeof(float) * c.vocab);
      if (logits_last && t == n - 1) memcpy(logits_last, logits.data(), sizeof(float) * c.vocab);
    }
  }
  return 0;
}

int orc_draft_step(const orc_model* m, orc_seq* ds, const float* h_prev, int32_t id, int numerics, float* h_out,
                   float* logits, int32_t draft_vocab) {
  const orc_config& c = m->c;
  if (!c.has_draft || !ds->draft) return -2;
  if (id < 0 || id >= c.vocab) return -1;
  const int H = c.n_embd, li = c.n_layer;
  const auto& sm = m->small[li];
  // nextn seed, embedding first (llm/mtp.go:352-384): res = eh_proj . concat(rms(e, enorm), rms(h, hnorm))
  std::vector<float> e(H), x(2 * H), h(H), xn(H);
  embed_row(*m, id, e.data());
  rmsnorm(e.data(), sm.enorm.data(), H, c.eps, x.data());
  rmsnorm(h_prev, sm.hnorm.data(), H, c.eps, x.data() + H);
  if (dev_like(numerics)) round_f16(x.data(), 2 * H);
  matvec(m->layers[li].eh_proj, 0, H, x.data(), h.data());
  Work w;
  int cell = ds->past, pos = ds->past + 1;  // the cell holds the token one position ahead of the trunk row that seeded it
  layer_token(*m, li, ds->l[0], h.data(), cell, pos, numerics, w, nullptr, nullptr, nullptr, nullptr, nullptr);
  ds->past++;
  if (h_out) memcpy(h_out, h.data(), sizeof(float) * H);
  if (logits) {
    rmsnorm(h.data(), sm.head_norm.data(), H, c.eps, xn.data());
    if (dev_like(numerics)) round_f16(xn.data(), H);
    int64_t nv = draft_vocab > 0 && draft_vocab < c.vocab ? draft_vocab : c.vocab;
    matvec(m->output, 0, nv, xn.data(), logits);
  }
  return 0;
}

}  // extern "C"
