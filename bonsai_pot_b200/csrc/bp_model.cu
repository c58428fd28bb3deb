// The engine around the attention path (include/bonsai_model.h): the model directory reader and
// validator (parse_config_ini / validate_cfg, src/model.rs:568-837), device residency of the Q1_0
// weights, the one-token and batched forward passes in the reference's dispatch order
// (src/forward.rs:578-672, 763-908, 975-1253), the sampler (src/session.rs:346-428) and the session
// loop (src/session.rs:162-344). Host code; every kernel it launches lives in bp_q1_ops.cu or in the
// attention files.
#include <errno.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <limits>
#include <map>
#include <new>
#include <string>
#include <type_traits>
#include <vector>

#include "../../include/bonsai_model.h"
#include "bp_common.cuh"
#include "bp_q1_ops.cuh"

namespace {

constexpr uint32_t M_MAX = 512;     // src/model.rs:502
constexpr uint32_t TOPK_MAX = 32;   // src/model.rs:279

struct TensorEntry {  // a manifest section of config.ini (src/model.rs:586-606)
  std::string dtype, buffer;
  std::vector<uint64_t> shape;
  uint64_t offset = 0, length = 0, d_offset = 0, qs_offset = 0, nb = 0;
};

struct Config {
  uint32_t n_layer = 0, n_embd = 0, n_ff = 0, n_head = 0, n_kv_head = 0, head_dim = 0, n_vocab = 0, eos_token_id = 0;
  uint32_t rope_orig_context = 0, n_kv_groups = 0, q_dim = 0, kv_dim = 0;
  float rope_freq_base = 0.f, rms_eps = 0.f;
  bool add_bos = false, tied_embeddings = false;
  std::map<std::string, TensorEntry> manifest;
};

struct Fail {
  int status;
  std::string msg;
};
#define CFG_FAIL(text) return Fail{BP_ERR_CONFIG, std::string("invalid config: ") + (text)}

std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
  return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}

template <typename T>
bool parse_num(const std::string& s, T* out) {
  if (s.empty()) return false;
  errno = 0;
  char* end = nullptr;
  if constexpr (std::is_floating_point<T>::value) {
    const double v = strtod(s.c_str(), &end);
    if (errno || *end) return false;
    *out = static_cast<T>(v);
  } else {
    if (s[0] == '-') return false;
    const unsigned long long v = strtoull(s.c_str(), &end, 10);
    if (errno || *end || v > static_cast<unsigned long long>(std::numeric_limits<T>::max())) return false;
    *out = static_cast<T>(v);
  }
  return true;
}

// parse_config_ini (src/model.rs:568-656): `key = value` globals, then `[tensor]` sections.
Fail parse_config_ini(const std::string& text, Config* cfg) {
  std::map<std::string, std::string> globals, fields;
  std::string section;
  bool in_section = false;
  auto build_entry = [&](TensorEntry* e) -> Fail {
    auto get = [&](const char* k, std::string* v) {
      auto it = fields.find(k);
      if (it == fields.end()) return false;
      *v = it->second;
      return true;
    };
    std::string shape;
    if (!get("shape", &shape) || !get("dtype", &e->dtype) || !get("buffer", &e->buffer)) CFG_FAIL("config.ini missing required field");
    size_t pos = 0;
    while (pos <= shape.size()) {
      const size_t comma = shape.find(',', pos);
      const std::string item = shape.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
      uint64_t v;
      if (!parse_num(item, &v)) CFG_FAIL("config.ini shape has invalid value");
      e->shape.push_back(v);
      if (comma == std::string::npos) break;
      pos = comma + 1;
    }
    std::string s;
    if (!get("offset", &s)) CFG_FAIL("config.ini missing required field");
    if (!parse_num(s, &e->offset)) CFG_FAIL("config.ini field has invalid value");
    if (!get("length", &s)) CFG_FAIL("config.ini missing required field");
    if (!parse_num(s, &e->length)) CFG_FAIL("config.ini field has invalid value");
    const std::pair<const char*, uint64_t*> opt[] = {{"d_offset", &e->d_offset}, {"qs_offset", &e->qs_offset}, {"nb", &e->nb}};
    for (auto& o : opt)
      if (get(o.first, &s) && !parse_num(s, o.second)) CFG_FAIL("config.ini field has invalid value");
    return Fail{BP_OK, ""};
  };
  size_t pos = 0;
  while (pos <= text.size()) {
    const size_t nl = text.find('\n', pos);
    const std::string line = trim(text.substr(pos, nl == std::string::npos ? std::string::npos : nl - pos));
    pos = nl == std::string::npos ? text.size() + 1 : nl + 1;
    if (line.empty()) continue;
    if (line.size() >= 2 && line.front() == '[' && line.back() == ']') {
      if (in_section) {
        TensorEntry e;
        Fail f = build_entry(&e);
        if (f.status) return f;
        cfg->manifest[section] = e;
        fields.clear();
      }
      section = line.substr(1, line.size() - 2);
      in_section = true;
    } else {
      const size_t eq = line.find(" = ");
      if (eq == std::string::npos) continue;
      (in_section ? fields : globals)[line.substr(0, eq)] = line.substr(eq + 3);
    }
  }
  if (in_section) {
    TensorEntry e;
    Fail f = build_entry(&e);
    if (f.status) return f;
    cfg->manifest[section] = e;
  }
  auto u32 = [&](const char* k, uint32_t* out) -> Fail {
    auto it = globals.find(k);
    if (it == globals.end()) CFG_FAIL("config.ini missing required field");
    if (!parse_num(it->second, out)) CFG_FAIL("config.ini field has invalid value");
    return Fail{BP_OK, ""};
  };
  auto f32 = [&](const char* k, float* out) -> Fail {
    auto it = globals.find(k);
    if (it == globals.end()) CFG_FAIL("config.ini missing required field");
    if (!parse_num(it->second, out)) CFG_FAIL("config.ini field has invalid value");
    return Fail{BP_OK, ""};
  };
  auto flag = [&](const char* k, bool* out) -> Fail {
    auto it = globals.find(k);
    if (it == globals.end()) CFG_FAIL("config.ini missing required field");
    *out = it->second == "true";
    return Fail{BP_OK, ""};
  };
  const std::pair<const char*, uint32_t*> ints[] = {
      {"n_layer", &cfg->n_layer}, {"n_embd", &cfg->n_embd}, {"n_ff", &cfg->n_ff}, {"n_head", &cfg->n_head},
      {"n_kv_head", &cfg->n_kv_head}, {"head_dim", &cfg->head_dim}};
  for (auto& i : ints) { Fail f = u32(i.first, i.second); if (f.status) return f; }
  { Fail f = f32("rope_freq_base", &cfg->rope_freq_base); if (f.status) return f; }
  { Fail f = f32("rms_eps", &cfg->rms_eps); if (f.status) return f; }
  const std::pair<const char*, uint32_t*> ints2[] = {{"n_vocab", &cfg->n_vocab}, {"eos_token_id", &cfg->eos_token_id}};
  for (auto& i : ints2) { Fail f = u32(i.first, i.second); if (f.status) return f; }
  { Fail f = flag("add_bos", &cfg->add_bos); if (f.status) return f; }
  const std::pair<const char*, uint32_t*> ints3[] = {{"rope_orig_context", &cfg->rope_orig_context}, {"n_kv_groups", &cfg->n_kv_groups},
                                                     {"q_dim", &cfg->q_dim}, {"kv_dim", &cfg->kv_dim}};
  for (auto& i : ints3) { Fail f = u32(i.first, i.second); if (f.status) return f; }
  { Fail f = flag("tied_embeddings", &cfg->tied_embeddings); if (f.status) return f; }
  return Fail{BP_OK, ""};
}

uint64_t pad4(uint64_t n) { return (n + 3) & ~3ull; }

// validate_cfg (src/model.rs:658-837), with its messages.
Fail validate_cfg(const Config& c) {
  if (c.add_bos) CFG_FAIL("config: add_bos=true but the runtime never prepends BOS; re-extract with a supported model");
  if (c.rope_orig_context == 0) CFG_FAIL("config: rope_orig_context must be > 0");
  if (c.n_kv_head == 0 || c.n_head % c.n_kv_head != 0) CFG_FAIL("config: n_head must be divisible by n_kv_head");
  if (c.n_kv_groups != c.n_head / c.n_kv_head) CFG_FAIL("config: n_kv_groups != n_head / n_kv_head");
  if (c.q_dim != c.n_head * c.head_dim) CFG_FAIL("config: q_dim != n_head * head_dim");
  if (c.kv_dim != c.n_kv_head * c.head_dim) CFG_FAIL("config: kv_dim != n_kv_head * head_dim");
  struct Spec { const char* tag; const char* dtype; std::vector<uint64_t> shape; const char* buffer; };
  const uint64_t e = c.n_embd, ff = c.n_ff, q = c.q_dim, kv = c.kv_dim, v = c.n_vocab, hd = c.head_dim;
  const Spec layer_specs[] = {
      {"attn_q.weight", "Q1_0", {e, q}, "weights_attn.bin"},        {"attn_k.weight", "Q1_0", {e, kv}, "weights_attn.bin"},
      {"attn_v.weight", "Q1_0", {e, kv}, "weights_attn.bin"},       {"attn_output.weight", "Q1_0", {q, e}, "weights_attn.bin"},
      {"ffn_gate.weight", "Q1_0", {e, ff}, "weights_ffn_gate_up.bin"}, {"ffn_up.weight", "Q1_0", {e, ff}, "weights_ffn_gate_up.bin"},
      {"ffn_down.weight", "Q1_0", {ff, e}, "weights_ffn_down.bin"}, {"attn_norm.weight", "F16", {e}, "weights_norms.bin"},
      {"attn_q_norm.weight", "F16", {hd}, "weights_norms.bin"},     {"attn_k_norm.weight", "F16", {hd}, "weights_norms.bin"},
      {"ffn_norm.weight", "F16", {e}, "weights_norms.bin"}};
  auto check = [&](const std::string& name, const Spec& s) -> Fail {
    auto it = c.manifest.find(name);
    if (it == c.manifest.end()) CFG_FAIL("manifest: expected tensor missing (re-extract the model dir)");
    const TensorEntry& t = it->second;
    if (t.dtype != s.dtype) CFG_FAIL("manifest: tensor has wrong dtype");
    if (t.shape != s.shape) CFG_FAIL("manifest: tensor has wrong shape");
    if (t.buffer != s.buffer) CFG_FAIL("manifest: tensor is in wrong buffer file");
    if (t.dtype == "Q1_0") {
      const uint64_t n_in = s.shape[0], n_out = s.shape.size() > 1 ? s.shape[1] : 1;
      if (n_in % 128 != 0) CFG_FAIL("manifest: Q1_0 tensor n_in not divisible by 128");
      const uint64_t nb = n_in / 128;
      if (t.nb != nb) CFG_FAIL("manifest: Q1_0 tensor nb != n_in/128");
      if (t.qs_offset != pad4(t.d_offset + n_out * nb * 2)) CFG_FAIL("manifest: Q1_0 tensor qs_offset != pad4(d_offset + n_out*nb*2)");
      if (t.length != (t.qs_offset - t.d_offset) + pad4(n_out * nb * 16)) CFG_FAIL("manifest: Q1_0 tensor length mismatch");
    } else if (t.dtype == "F16") {
      uint64_t prod = 1;
      for (uint64_t d : s.shape) prod *= d;
      if (t.length != pad4(prod * 2)) CFG_FAIL("manifest: F16 tensor length mismatch");
    } else {
      CFG_FAIL("manifest: unknown dtype");
    }
    return Fail{BP_OK, ""};
  };
  for (uint32_t il = 0; il < c.n_layer; il++)
    for (const Spec& s : layer_specs) {
      Fail f = check("blk." + std::to_string(il) + "." + s.tag, s);
      if (f.status) return f;
    }
  {
    Fail f = check("output_norm.weight", Spec{"", "F16", {e}, "weights_norms.bin"});
    if (f.status) return f;
    f = check("token_embd.weight", Spec{"", "Q1_0", {e, v}, "weights_embed_lmhead.bin"});
    if (f.status) return f;
    if (!c.tied_embeddings) {
      f = check("output.weight", Spec{"", "Q1_0", {e, v}, "weights_embed_lmhead.bin"});
      if (f.status) return f;
    }
  }
  return Fail{BP_OK, ""};
}

Fail read_file(const std::string& path, std::vector<uint8_t>* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return Fail{BP_ERR_IO, "io error reading " + path + ": " + strerror(errno)};
  fseek(f, 0, SEEK_END);
  const long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  out->resize(n > 0 ? static_cast<size_t>(n) : 0);
  const size_t got = out->empty() ? 0 : fread(out->data(), 1, out->size(), f);
  fclose(f);
  if (got != out->size()) return Fail{BP_ERR_IO, "io error reading " + path + ": short read"};
  return Fail{BP_OK, ""};
}

Fail load_config(const std::string& dir, Config* cfg) {
  std::vector<uint8_t> text;
  Fail f = read_file(dir + "/config.ini", &text);
  if (f.status) return f;
  f = parse_config_ini(std::string(text.begin(), text.end()), cfg);
  if (f.status) return f;
  return validate_cfg(*cfg);
}

}  // namespace

// ---------------------------------------------------------------------------------------------
struct LayerTensors {
  bp_q1_tensor wq, wk, wv, wo, wg, wu, wd;
  const __half *attn_norm, *q_norm, *k_norm, *ffn_norm;
};

struct bp_model {
  Config cfg;
  uint32_t max_seq = 0;
  int device = 0;
  std::string msg;
  bp_error_detail detail = {};
  bp_attn_ctx* attn = nullptr;
  cudaStream_t stream = nullptr;
  uint8_t* dev_file[5] = {};   // the weight files as they are on disk
  void* dev_bits[4] = {};      // re-laid-out sign words: attn, gate_up, down, embed_lmhead (same offsets as the files' qs regions)
  std::vector<LayerTensors> layers;
  bp_q1_tensor embed, lm_head;
  const __half* output_norm = nullptr;
  // activations (ActLayout, src/model.rs:287-333), f16 [m_max][...] each
  __half *x = nullptr, *x_norm = nullptr, *q = nullptr, *k_cur = nullptr, *v_cur = nullptr, *attn_out = nullptr, *gate = nullptr,
         *up = nullptr, *ffn_in = nullptr, *logits = nullptr, *q_roped = nullptr;
  float* a_d = nullptr;        // Q8_0 activations: scales [m_max][n_ff / 32]
  int8_t* a_qs = nullptr;      //                  quants [m_max][n_ff]
  uint32_t* tokens_dev = nullptr;
  float* topk_val = nullptr;
  uint32_t* topk_idx = nullptr;
  uint32_t tap_mode = 0;
  uint8_t* tap_buf = nullptr;
  // The one-token step as a CUDA graph (token copy, embed, layers, output suffix, result copies). The only
  // launches whose arguments depend on the position are the attention calls: their nodes are patched per step
  // with what the attention library's launcher produces for the new position.
  struct StepGraph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<std::vector<bp_launch_record>> attn;  // per layer: the attention launches as captured
    bp_launch_recorder patch;                         // the recorder of the per-step pass
    bool valid = false;
  } sg;
  bool step_graph = true;     // bp_model_set_step_graph
  uint64_t graph_steps = 0;   // steps that ran as a graph launch
  uint32_t* token_pin = nullptr;  // pinned: the token of the step (read by the graph's copy node)
  float* res_val_pin = nullptr;   // pinned: top-k results of the step
  uint32_t* res_idx_pin = nullptr;
};

struct bp_session {
  bp_model* m;
  uint32_t pos;
};

namespace {

int mfail(bp_model* m, int status, const std::string& msg, uint32_t pos = 0, uint32_t n = 0, uint32_t max = 0, int cuda_error = 0) {
  if (m) {
    m->msg = msg;
    m->detail = bp_error_detail{status, pos, n, max, cuda_error};
  }
  return status;
}
int mfail_cuda(bp_model* m, cudaError_t e, const char* where) {
  return mfail(m, BP_ERR_CUDA, std::string("CUDA error in ") + where + ": " + cudaGetErrorString(e), 0, 0, 0, static_cast<int>(e));
}
#define M_CUDA(m, call)                                      \
  do {                                                       \
    cudaError_t e_ = (call);                                 \
    if (e_ != cudaSuccess) return mfail_cuda(m, e_, #call);  \
  } while (0)
// a status of the attention context, with its message
int attn_status(bp_model* m, int st) {
  if (st == BP_OK) return BP_OK;
  bp_error_detail d;
  bp_last_error_detail(m->attn, &d);
  m->msg = bp_last_error_message(m->attn);
  m->detail = d;
  return st;
}
// check_device (src/model.rs:1733-1741): a latched status of the attention context (lost device, a
// device-side wait that ran out) fails every model and session call from then on.
int device_status(bp_model* m) {
  const int st = bp_ctx_status(m->attn);
  if (st == BP_OK) return BP_OK;
  return mfail(m, st, st == BP_ERR_TIMEOUT ? "a bounded device-side wait gave up: the model is unusable, load it again"
                                           : "device lost: the model is unusable, load it again");
}
int model_enter(bp_model* m) {
  if (!m) return BP_ERR_NULL;
  if (!m->attn) return mfail(m, BP_ERR_CONFIG, "invalid config: model is not loaded");
  return device_status(m);
}

const int FILE_OF_BITS[5] = {0, 1, 2, -1, 3};
const char* const FILE_NAMES[5] = {"weights_attn.bin", "weights_ffn_gate_up.bin", "weights_ffn_down.bin", "weights_norms.bin",
                                   "weights_embed_lmhead.bin"};
int file_index(const std::string& name) {
  for (int i = 0; i < 5; i++)
    if (name == FILE_NAMES[i]) return i;
  return -1;
}

bp_q1_tensor q1_view(const bp_model* m, const std::string& name) {
  const TensorEntry& t = m->cfg.manifest.at(name);
  const int fi = file_index(t.buffer), bi = FILE_OF_BITS[fi];
  bp_q1_tensor w;
  w.d = reinterpret_cast<const __half*>(m->dev_file[fi] + t.d_offset);
  w.qs = m->dev_file[fi] + t.qs_offset;
  w.bits = static_cast<const uint8_t*>(m->dev_bits[bi]) + t.qs_offset;
  w.k = static_cast<uint32_t>(t.shape[0]);
  w.n = static_cast<uint32_t>(t.shape.size() > 1 ? t.shape[1] : 1);
  return w;
}
const __half* f16_view(const bp_model* m, const std::string& name) {
  const TensorEntry& t = m->cfg.manifest.at(name);
  return reinterpret_cast<const __half*>(m->dev_file[file_index(t.buffer)] + t.offset);
}

// The attention call of layer il at position pos (Q norm + RoPE, cache write, attention: one launch by default).
cudaError_t attention_call(bp_model* m, uint32_t il, uint32_t pos) {
  const LayerTensors& lt = m->layers[il];
  uint32_t launches = 0;
  return bp_launch_decode_fused(m->attn, m->stream, il, m->q, m->q_roped, lt.q_norm, m->k_cur, m->v_cur, lt.k_norm, pos, m->attn_out,
                                &launches);
}

// One layer of the one-token path: layer_pre_kv_in_pass, dispatch_kv_writeback_fused, layer_post_kv_in_pass
// (src/forward.rs:608-631, 763-908). The three attention dispatches are one call of the attention library.
// in_graph: the launches are being captured into the step's graph (attn_nodes then receives the attention
// launches with their nodes); the choice of dependent launches differs between the two ways of launching.
// Which launches carry programmatic stream serialization was measured per kernel on the 8B shape (us per layer,
// stream launches / graph replay): all four matvecs 55.0 / 53.2, all but the down projection 48.8 / 44.8, gate + up
// only 49.9 / 41.1, none 51.2 / 42.3. The down projection's CTAs, resident early, take the SM slots that the
// second wave of the gate + up launch is waiting for.
int decode_layer(bp_model* m, uint32_t il, uint32_t pos, bool in_graph = false, std::vector<bp_launch_record>* attn_nodes = nullptr) {
  const Config& c = m->cfg;
  const LayerTensors& lt = m->layers[il];
  cudaStream_t s = m->stream;
  const bool pdl = !in_graph;
  {
    const bp_q1_tensor w[3] = {lt.wq, lt.wk, lt.wv};
    __half* const out[3] = {m->q, m->k_cur, m->v_cur};
    M_CUDA(m, bp_q1_matvec_normed(pdl, s, w, out, 3, m->x, lt.attn_norm, c.rms_eps));
  }
  if (attn_nodes != nullptr) {  // capturing: keep the nodes of the attention launches
    bp_launch_recorder rec;
    rec.mode = 2;
    bp_recorder() = &rec;
    const cudaError_t e = attention_call(m, il, pos);
    bp_recorder() = nullptr;
    M_CUDA(m, e);
    *attn_nodes = std::move(rec.records);
  } else {
    M_CUDA(m, attention_call(m, il, pos));
  }
  if (m->tap_mode) {
    uint8_t* slot = m->tap_buf + static_cast<size_t>(il) * c.q_dim * 2;
    if (m->tap_mode == 1) {
      M_CUDA(m, cudaMemcpyAsync(slot, m->attn_out, static_cast<size_t>(c.q_dim) * 2, cudaMemcpyDeviceToHost, s));
    } else {
      M_CUDA(m, cudaMemcpyAsync(m->attn_out, slot, static_cast<size_t>(c.q_dim) * 2, cudaMemcpyHostToDevice, s));
    }
  }
  M_CUDA(m, bp_q1_matvec(pdl, s, lt.wo, m->attn_out, m->x, true));
  // matvec_q1_0_fused_normed over (gate, up) and silu(gate) * up in one launch: a lane computes row i of both
  // tensors and writes the f16 value that feeds the down projection (the same values dispatch_matvec_q1_0_silu
  // stages; that shader as one kernel had each of the 256 CTAs of the 4096-row down tensor recompute all 12288
  // of them: 27.6 us against 8 for the plain matvec).
  M_CUDA(m, bp_q1_matvec_normed_silu(true, s, lt.wg, lt.wu, m->ffn_in, m->x, lt.ffn_norm, c.rms_eps));
  M_CUDA(m, bp_q1_matvec(false, s, lt.wd, m->ffn_in, m->x, true));
  return BP_OK;
}

// output_norm (in place) + LM head + top-k over row `row` of x, then the k results to the host
// (the suffix of encode_step_matvec, src/forward.rs:632-670, and of prefill_matmul_topk, :1030-1058).
int output_suffix(bp_model* m, uint32_t row, uint32_t k, float* logits, uint32_t* indices) {
  const Config& c = m->cfg;
  cudaStream_t s = m->stream;
  __half* xr = m->x + static_cast<size_t>(row) * c.n_embd;
  M_CUDA(m, bp_q1_rms_norm(true, s, xr, xr, m->output_norm, c.n_embd, 1, c.rms_eps));
  M_CUDA(m, bp_q1_matvec(true, s, m->lm_head, xr, m->logits, false));
  M_CUDA(m, bp_q1_topk(true, s, m->logits, c.n_vocab, k, m->topk_val, m->topk_idx));
  M_CUDA(m, cudaMemcpyAsync(logits, m->topk_val, k * sizeof(float), cudaMemcpyDeviceToHost, s));
  M_CUDA(m, cudaMemcpyAsync(indices, m->topk_idx, k * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  M_CUDA(m, cudaStreamSynchronize(s));
  return device_status(m);
}

int step_no_suffix(bp_model* m, uint32_t token, uint32_t pos) {
  cudaStream_t s = m->stream;
  M_CUDA(m, cudaMemcpyAsync(m->tokens_dev, &token, sizeof token, cudaMemcpyHostToDevice, s));
  M_CUDA(m, bp_q1_embed(true, s, m->embed, m->tokens_dev, 1, m->x));
  for (uint32_t il = 0; il < m->cfg.n_layer; il++)
    if (int st = decode_layer(m, il, pos)) return st;
  return BP_OK;
}

void drop_step_graph(bp_model* m) {
  if (m->sg.exec) cudaGraphExecDestroy(m->sg.exec);
  if (m->sg.graph) cudaGraphDestroy(m->sg.graph);
  m->sg = bp_model::StepGraph();
}

// The whole step (token copy, embed, layers, output norm, LM head, top-k of TOPK_MAX, result copies) captured
// from the model's stream at position pos.
int capture_step_graph(bp_model* m, uint32_t pos) {
  const Config& c = m->cfg;
  cudaStream_t s = m->stream;
  drop_step_graph(m);
  m->sg.attn.resize(c.n_layer);
  M_CUDA(m, cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int st = BP_OK;
  cudaError_t e = cudaMemcpyAsync(m->tokens_dev, m->token_pin, sizeof(uint32_t), cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = bp_q1_embed(true, s, m->embed, m->tokens_dev, 1, m->x);
  for (uint32_t il = 0; e == cudaSuccess && st == BP_OK && il < c.n_layer; il++) st = decode_layer(m, il, pos, true, &m->sg.attn[il]);
  if (e == cudaSuccess && st == BP_OK) e = bp_q1_rms_norm(true, s, m->x, m->x, m->output_norm, c.n_embd, 1, c.rms_eps);
  if (e == cudaSuccess && st == BP_OK) e = bp_q1_matvec(true, s, m->lm_head, m->x, m->logits, false);
  if (e == cudaSuccess && st == BP_OK) e = bp_q1_topk(true, s, m->logits, c.n_vocab, TOPK_MAX, m->topk_val, m->topk_idx);
  if (e == cudaSuccess && st == BP_OK) e = cudaMemcpyAsync(m->res_val_pin, m->topk_val, TOPK_MAX * sizeof(float), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && st == BP_OK) e = cudaMemcpyAsync(m->res_idx_pin, m->topk_idx, TOPK_MAX * sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
  const cudaError_t e_end = cudaStreamEndCapture(s, &m->sg.graph);  // always: the stream must leave capture mode
  if (st != BP_OK) return st;
  M_CUDA(m, e);
  M_CUDA(m, e_end);
  M_CUDA(m, cudaGraphInstantiate(&m->sg.exec, m->sg.graph, 0));
  m->sg.valid = true;
  return BP_OK;
}

// The attention nodes of the captured step, patched for position pos. False: the launches no longer have the
// captured shape (another kernel instance, another number of launches): the step has to be captured again.
int patch_step_graph(bp_model* m, uint32_t pos, bool* ok) {
  *ok = false;
  for (uint32_t il = 0; il < m->cfg.n_layer; il++) {
    bp_launch_recorder& rec = m->sg.patch;  // its storage is reused from step to step
    rec.mode = 1;
    rec.records.clear();
    bp_recorder() = &rec;
    const cudaError_t e = attention_call(m, il, pos);
    bp_recorder() = nullptr;
    M_CUDA(m, e);
    const std::vector<bp_launch_record>& was = m->sg.attn[il];
    if (rec.records.size() != was.size()) return BP_OK;
    for (size_t i = 0; i < was.size(); i++) {
      bp_launch_record& r = rec.records[i];
      if (r.func != was[i].func) return BP_OK;
      void* argv[BP_RECORD_MAX_ARGS];
      if (r.overflow) return mfail(m, BP_ERR_CUDA, "an attention launch has more arguments than a launch record holds");
      for (uint32_t a = 0; a < r.n_args; a++) argv[a] = r.arg(a);
      cudaKernelNodeParams kp = {};
      kp.func = r.func;
      kp.gridDim = r.grid;
      kp.blockDim = r.block;
      kp.sharedMemBytes = static_cast<unsigned int>(r.smem);
      kp.kernelParams = argv;
      M_CUDA(m, cudaGraphExecKernelNodeSetParams(m->sg.exec, was[i].node, &kp));
    }
  }
  *ok = true;
  return BP_OK;
}

int step_topk_graph(bp_model* m, uint32_t token, uint32_t pos, uint32_t k, float* logits, uint32_t* indices) {
  *m->token_pin = token;
  bool patched = false;
  if (m->sg.valid)
    if (int st = patch_step_graph(m, pos, &patched)) return st;
  if (!patched)
    if (int st = capture_step_graph(m, pos)) return st;
  M_CUDA(m, cudaGraphLaunch(m->sg.exec, m->stream));
  M_CUDA(m, cudaStreamSynchronize(m->stream));
  m->graph_steps++;
  for (uint32_t i = 0; i < k; i++) {
    logits[i] = m->res_val_pin[i];
    indices[i] = m->res_idx_pin[i];
  }
  return device_status(m);
}

int quantize_and_matmul(bp_model* m, const __half* act, uint32_t k, uint32_t mt, const bp_q1_tensor* w, __half* const* out, uint32_t n_w,
                        bool accumulate) {
  cudaStream_t s = m->stream;
  M_CUDA(m, bp_q1_quantize_q8(true, s, act, k, mt, m->a_d, m->a_qs));
  M_CUDA(m, bp_q1_matmul_multi(true, s, w, out, n_w, mt, m->a_d, m->a_qs, accumulate, m->attn->err_dev, m->attn->opt_wait_limit));
  return BP_OK;
}

}  // namespace

extern "C" {

// ---- operators --------------------------------------------------------------------------------
#define OP_CUDA(call) ((call) == cudaSuccess ? BP_OK : BP_ERR_CUDA)
static bp_q1_tensor op_tensor(const void* d, const void* qs, const void* bits, uint32_t k, uint32_t n) {
  bp_q1_tensor w;
  w.d = static_cast<const __half*>(d);
  w.qs = static_cast<const uint8_t*>(qs);
  w.bits = bits;
  w.k = k;
  w.n = n;
  return w;
}
static bool bad_k(uint32_t k) { return k == 0 || k % 128u != 0; }

int bp_op_q1_relayout(void* stream, const void* qs, void* bits_out, uint64_t n_blocks) {
  if (!qs || !bits_out) return BP_ERR_NULL;
  if (n_blocks == 0) return BP_OK;
  return OP_CUDA(bp_q1_relayout(static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(qs), bits_out, n_blocks));
}
int bp_op_matvec_q1_0(void* stream, const void* d, const void* bits, uint32_t k, uint32_t n, const void* x, void* y, uint32_t accumulate) {
  if (!d || !bits || !x || !y) return BP_ERR_NULL;
  if (bad_k(k) || n == 0) return BP_ERR_CONFIG;
  return OP_CUDA(bp_q1_matvec(false, static_cast<cudaStream_t>(stream), op_tensor(d, nullptr, bits, k, n), static_cast<const __half*>(x),
                              static_cast<__half*>(y), accumulate != 0));
}
int bp_op_matvec_q1_0_fused_normed(void* stream, uint32_t k, const void* x, const void* w_norm, float eps, uint32_t n_ranges,
                                   const void* const* d, const void* const* bits, const uint32_t* n, void* const* out) {
  if (!x || !w_norm || !d || !bits || !n || !out) return BP_ERR_NULL;
  if (bad_k(k) || n_ranges == 0 || n_ranges > 3) return BP_ERR_CONFIG;
  bp_q1_tensor w[3];
  __half* o[3];
  for (uint32_t r = 0; r < n_ranges; r++) {
    if (!d[r] || !bits[r] || !out[r]) return BP_ERR_NULL;
    if (n[r] == 0 || n[r] % 16u != 0) return BP_ERR_CONFIG;
    w[r] = op_tensor(d[r], nullptr, bits[r], k, n[r]);
    o[r] = static_cast<__half*>(out[r]);
  }
  return OP_CUDA(bp_q1_matvec_normed(false, static_cast<cudaStream_t>(stream), w, o, n_ranges, static_cast<const __half*>(x),
                                     static_cast<const __half*>(w_norm), eps));
}
int bp_op_matvec_q1_0_silu(void* stream, const void* d, const void* bits, uint32_t k, uint32_t n, const void* gate, const void* up, void* y,
                           uint32_t accumulate) {
  if (!d || !bits || !gate || !up || !y) return BP_ERR_NULL;
  if (bad_k(k) || n == 0) return BP_ERR_CONFIG;
  return OP_CUDA(bp_q1_matvec_silu(false, static_cast<cudaStream_t>(stream), op_tensor(d, nullptr, bits, k, n),
                                   static_cast<const __half*>(gate), static_cast<const __half*>(up), static_cast<__half*>(y), accumulate != 0));
}
void bp_op_set_matvec_rows(uint32_t rows_per_lane) {
  const uint32_t r = rows_per_lane & 7u;
  bp_q1_set_matvec_rows(rows_per_lane < 16 && (r == 0 || r == 1 || r == 2 || r == 4) ? rows_per_lane : 0);
}
int bp_op_rms_norm(void* stream, const void* in, void* out, const void* w, uint32_t group_size, uint32_t n_groups, float eps) {
  if (!in || !out || !w) return BP_ERR_NULL;
  if (group_size == 0 || n_groups == 0) return BP_ERR_CONFIG;
  return OP_CUDA(bp_q1_rms_norm(false, static_cast<cudaStream_t>(stream), static_cast<const __half*>(in), static_cast<__half*>(out),
                                static_cast<const __half*>(w), group_size, n_groups, eps));
}
int bp_op_silu_mul(void* stream, const void* gate, const void* up, void* out, uint64_t n) {
  if (!gate || !up || !out) return BP_ERR_NULL;
  if (n == 0) return BP_OK;
  return OP_CUDA(bp_q1_silu_mul(false, static_cast<cudaStream_t>(stream), static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                static_cast<__half*>(out), n));
}
int bp_op_embed(void* stream, const void* d, const void* qs, uint32_t k, const void* tokens, uint32_t m, void* x) {
  if (!d || !qs || !tokens || !x) return BP_ERR_NULL;
  if (bad_k(k)) return BP_ERR_CONFIG;
  if (m == 0) return BP_OK;
  return OP_CUDA(bp_q1_embed(false, static_cast<cudaStream_t>(stream), op_tensor(d, qs, nullptr, k, 0), static_cast<const uint32_t*>(tokens), m,
                             static_cast<__half*>(x)));
}
int bp_op_quantize_q8_0(void* stream, const void* x, uint32_t k, uint32_t m, void* d_out, void* qs_out) {
  if (!x || !d_out || !qs_out) return BP_ERR_NULL;
  if (k == 0 || k % 32u != 0) return BP_ERR_CONFIG;
  if (m == 0) return BP_OK;
  return OP_CUDA(bp_q1_quantize_q8(false, static_cast<cudaStream_t>(stream), static_cast<const __half*>(x), k, m, static_cast<float*>(d_out),
                                   static_cast<int8_t*>(qs_out)));
}
int bp_op_matmul_q1_0_q8_0(void* stream, const void* d, const void* qs, uint32_t k, uint32_t n, uint32_t m, const void* a_d, const void* a_qs,
                           void* y, uint32_t accumulate) {
  if (!d || !qs || !a_d || !a_qs || !y) return BP_ERR_NULL;
  if (bad_k(k) || n == 0) return BP_ERR_CONFIG;
  if (m == 0) return BP_OK;
  return OP_CUDA(bp_q1_matmul(false, static_cast<cudaStream_t>(stream), op_tensor(d, qs, nullptr, k, n), m, static_cast<const float*>(a_d),
                              static_cast<const int8_t*>(a_qs), static_cast<__half*>(y), accumulate != 0));
}
void bp_op_set_matmul_variant(uint32_t variant) { bp_q1_set_matmul_variant(variant); }
int bp_op_device_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return BP_ERR_CUDA;
  uint32_t code = 0;
  if (bp_q1_take_error(&code) != cudaSuccess) return BP_ERR_CUDA;
  return code != 0 ? BP_ERR_TIMEOUT : BP_OK;
}
int bp_op_topk_reduce(void* stream, const void* logits, uint32_t n, uint32_t k, void* out_val, void* out_idx) {
  if (!logits || !out_val || !out_idx) return BP_ERR_NULL;
  if (n == 0 || k == 0) return BP_ERR_CONFIG;
  return OP_CUDA(bp_q1_topk(false, static_cast<cudaStream_t>(stream), static_cast<const __half*>(logits), n, k, static_cast<float*>(out_val),
                            static_cast<uint32_t*>(out_idx)));
}

// ---- model ---------------------------------------------------------------------------------------
int bp_model_check_dir(const char* dir, char* msg, size_t msg_len) {
  if (!dir) return BP_ERR_NULL;
  Config cfg;
  Fail f = load_config(dir, &cfg);
  if (msg && msg_len) snprintf(msg, msg_len, "%s", f.msg.c_str());
  return f.status;
}

int bp_model_load(const char* dir, uint32_t max_seq, int32_t device, bp_model** out) {
  if (!dir || !out) return BP_ERR_NULL;
  bp_model* m = new (std::nothrow) bp_model();
  *out = m;
  if (!m) return BP_ERR_CUDA;
  if (max_seq == 0) return mfail(m, BP_ERR_CONFIG, "invalid config: max_seq must be > 0");
  {
    Fail f = load_config(dir, &m->cfg);
    if (f.status) return mfail(m, f.status, f.msg);
  }
  const Config& c = m->cfg;
  m->max_seq = max_seq;
  m->device = device;
  // the fused matvec's ranges must be multiples of 16 rows (matvec_q1_0_fused_normed.wgsl:22-24)
  if (c.q_dim % 16 || c.kv_dim % 16 || c.n_ff % 16) return mfail(m, BP_ERR_CONFIG, "invalid config: q_dim, kv_dim and n_ff must be multiples of 16");
  bp_attn_config ac = {};
  ac.n_layer = c.n_layer;
  ac.n_head = c.n_head;
  ac.n_kv_head = c.n_kv_head;
  ac.head_dim = c.head_dim;
  ac.max_seq = max_seq;
  ac.rms_eps = c.rms_eps;
  ac.rope_freq_base = c.rope_freq_base;
  ac.max_prefill = M_MAX;
  ac.n_shards = 1;
  ac.shard = 0;
  ac.device = device;
  {
    const int st = bp_attn_create(&ac, &m->attn);
    if (st != BP_OK) {
      const int r = attn_status(m, st);
      bp_attn_destroy(m->attn);
      m->attn = nullptr;
      return r;
    }
  }
  M_CUDA(m, cudaSetDevice(device));
  M_CUDA(m, cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  for (int fi = 0; fi < 5; fi++) {
    std::vector<uint8_t> bytes;
    Fail f = read_file(std::string(dir) + "/" + FILE_NAMES[fi], &bytes);
    if (f.status) return mfail(m, f.status, f.msg);
    for (const auto& kv : c.manifest)
      if (kv.second.buffer == FILE_NAMES[fi] && kv.second.offset + kv.second.length > bytes.size())
        return mfail(m, BP_ERR_CONFIG, "invalid config: manifest: tensor extends past the end of its buffer file");
    M_CUDA(m, cudaMalloc(&m->dev_file[fi], bytes.size() + 16));
    M_CUDA(m, cudaMemcpy(m->dev_file[fi], bytes.data(), bytes.size(), cudaMemcpyHostToDevice));
    if (FILE_OF_BITS[fi] >= 0) M_CUDA(m, cudaMalloc(&m->dev_bits[FILE_OF_BITS[fi]], bytes.size() + 16));
  }
  // sign words of every Q1_0 tensor in the matvec kernels' layout, at the same offsets as the originals
  for (const auto& kv : c.manifest) {
    const TensorEntry& t = kv.second;
    if (t.dtype != "Q1_0") continue;
    const int fi = file_index(t.buffer);
    if (t.qs_offset % 16 != 0) return mfail(m, BP_ERR_CONFIG, "invalid config: manifest: Q1_0 sign region is not 16-byte aligned");
    const uint64_t n_out = t.shape.size() > 1 ? t.shape[1] : 1;
    M_CUDA(m, bp_q1_relayout(m->stream, m->dev_file[fi] + t.qs_offset, static_cast<uint8_t*>(m->dev_bits[FILE_OF_BITS[fi]]) + t.qs_offset,
                             n_out * t.nb));
  }
  m->layers.resize(c.n_layer);
  for (uint32_t il = 0; il < c.n_layer; il++) {
    const std::string p = "blk." + std::to_string(il) + ".";
    LayerTensors& lt = m->layers[il];
    lt.wq = q1_view(m, p + "attn_q.weight");
    lt.wk = q1_view(m, p + "attn_k.weight");
    lt.wv = q1_view(m, p + "attn_v.weight");
    lt.wo = q1_view(m, p + "attn_output.weight");
    lt.wg = q1_view(m, p + "ffn_gate.weight");
    lt.wu = q1_view(m, p + "ffn_up.weight");
    lt.wd = q1_view(m, p + "ffn_down.weight");
    lt.attn_norm = f16_view(m, p + "attn_norm.weight");
    lt.q_norm = f16_view(m, p + "attn_q_norm.weight");
    lt.k_norm = f16_view(m, p + "attn_k_norm.weight");
    lt.ffn_norm = f16_view(m, p + "ffn_norm.weight");
  }
  m->embed = q1_view(m, "token_embd.weight");
  m->lm_head = c.tied_embeddings ? m->embed : q1_view(m, "output.weight");
  m->output_norm = f16_view(m, "output_norm.weight");
  const size_t mm = M_MAX;
  M_CUDA(m, cudaMalloc(&m->x, mm * c.n_embd * 2));
  M_CUDA(m, cudaMalloc(&m->x_norm, mm * c.n_embd * 2));
  M_CUDA(m, cudaMalloc(&m->q, mm * c.q_dim * 2));
  M_CUDA(m, cudaMalloc(&m->q_roped, static_cast<size_t>(c.q_dim) * 2));
  M_CUDA(m, cudaMalloc(&m->k_cur, mm * c.kv_dim * 2));
  M_CUDA(m, cudaMalloc(&m->v_cur, mm * c.kv_dim * 2));
  M_CUDA(m, cudaMalloc(&m->attn_out, mm * c.q_dim * 2));
  M_CUDA(m, cudaMalloc(&m->gate, mm * c.n_ff * 2));
  M_CUDA(m, cudaMalloc(&m->up, mm * c.n_ff * 2));
  M_CUDA(m, cudaMalloc(&m->ffn_in, mm * c.n_ff * 2));
  M_CUDA(m, cudaMalloc(&m->logits, (static_cast<size_t>(c.n_vocab) + 2) * 2));
  const uint32_t k_max = c.n_ff > c.q_dim ? (c.n_ff > c.n_embd ? c.n_ff : c.n_embd) : (c.q_dim > c.n_embd ? c.q_dim : c.n_embd);
  M_CUDA(m, cudaMalloc(&m->a_d, mm * (k_max / 32) * sizeof(float)));
  M_CUDA(m, cudaMalloc(&m->a_qs, mm * k_max));
  M_CUDA(m, cudaMalloc(&m->tokens_dev, mm * sizeof(uint32_t)));
  M_CUDA(m, cudaMalloc(&m->topk_val, TOPK_MAX * sizeof(float)));
  M_CUDA(m, cudaMalloc(&m->topk_idx, TOPK_MAX * sizeof(uint32_t)));
  M_CUDA(m, cudaMallocHost(&m->token_pin, sizeof(uint32_t)));
  M_CUDA(m, cudaMallocHost(&m->res_val_pin, TOPK_MAX * sizeof(float)));
  M_CUDA(m, cudaMallocHost(&m->res_idx_pin, TOPK_MAX * sizeof(uint32_t)));
  M_CUDA(m, cudaStreamSynchronize(m->stream));
  return BP_OK;
}

void bp_model_free(bp_model* m) {
  if (!m) return;
  if (m->stream) {
    cudaSetDevice(m->device);
    cudaStreamSynchronize(m->stream);
  }
  for (auto p : m->dev_file) cudaFree(p);
  for (auto p : m->dev_bits) cudaFree(p);
  void* bufs[] = {m->x, m->x_norm, m->q, m->q_roped, m->k_cur, m->v_cur, m->attn_out, m->gate, m->up, m->ffn_in, m->logits,
                  m->a_d, m->a_qs, m->tokens_dev, m->topk_val, m->topk_idx};
  for (void* p : bufs) cudaFree(p);
  drop_step_graph(m);
  cudaFreeHost(m->token_pin);
  cudaFreeHost(m->res_val_pin);
  cudaFreeHost(m->res_idx_pin);
  if (m->stream) cudaStreamDestroy(m->stream);
  bp_attn_destroy(m->attn);
  delete m;
}

int bp_model_get_config(const bp_model* m, bp_model_config* out) {
  if (!m || !out) return BP_ERR_NULL;
  const Config& c = m->cfg;
  *out = bp_model_config{c.n_layer, c.n_embd, c.n_ff, c.n_head, c.n_kv_head, c.head_dim, c.n_vocab, c.eos_token_id, c.q_dim, c.kv_dim,
                         c.rope_freq_base, c.rms_eps, c.tied_embeddings ? 1u : 0u, m->max_seq, M_MAX};
  return BP_OK;
}
const char* bp_model_last_error(const bp_model* m) { return m ? m->msg.c_str() : ""; }
void bp_model_error_detail(const bp_model* m, bp_error_detail* out) {
  if (m && out) *out = m->detail;
}
bp_attn_ctx* bp_model_attn(bp_model* m) { return m ? m->attn : nullptr; }

int bp_model_step_topk(bp_model* m, uint32_t token, uint32_t pos, uint32_t k, float* logits, uint32_t* indices) {
  if (int st = model_enter(m)) return st;
  if (!logits || !indices) return mfail(m, BP_ERR_NULL, "null pointer argument");
  if (token >= m->cfg.n_vocab) return mfail(m, BP_ERR_CONFIG, "invalid config: token id out of range");
  if (static_cast<uint64_t>(pos) + 1 > m->max_seq) {
    char buf[160];
    snprintf(buf, sizeof buf, "context overflow: pos %u + tokens %u > max_seq %u", pos, 1u, m->max_seq);
    return mfail(m, BP_ERR_CONTEXT_OVERFLOW, buf, pos, 1, m->max_seq);
  }
  k = k < 1 ? 1 : (k > TOPK_MAX ? TOPK_MAX : k);
  M_CUDA(m, cudaSetDevice(m->device));
  // as a graph when every launch of the attention call goes through bp_launch (the tcgen05 decode path does)
  if (m->step_graph && m->tap_mode == 0 && bp_use_umma(m->attn)) return step_topk_graph(m, token, pos, k, logits, indices);
  if (int st = step_no_suffix(m, token, pos)) return st;
  return output_suffix(m, 0, k, logits, indices);
}

int bp_model_set_step_graph(bp_model* m, uint32_t enable) {
  if (int st = model_enter(m)) return st;
  m->step_graph = enable != 0;
  if (!m->step_graph) drop_step_graph(m);
  return BP_OK;
}
uint64_t bp_model_graph_steps(const bp_model* m) { return m ? m->graph_steps : 0; }

int bp_model_prefill_loop_topk(bp_model* m, const uint32_t* tokens, uint32_t n, uint32_t pos_base, uint32_t k, float* logits,
                               uint32_t* indices) {
  if (int st = model_enter(m)) return st;
  if (!tokens || !logits || !indices) return mfail(m, BP_ERR_NULL, "null pointer argument");
  if (n == 0) return mfail(m, BP_ERR_CONFIG, "invalid config: prefill needs at least one token");
  if (static_cast<uint64_t>(pos_base) + n > m->max_seq) {
    char buf[160];
    snprintf(buf, sizeof buf, "context overflow: pos %u + tokens %u > max_seq %u", pos_base, n, m->max_seq);
    return mfail(m, BP_ERR_CONTEXT_OVERFLOW, buf, pos_base, n, m->max_seq);
  }
  for (uint32_t i = 0; i < n; i++)
    if (tokens[i] >= m->cfg.n_vocab) return mfail(m, BP_ERR_CONFIG, "invalid config: token id out of range");
  M_CUDA(m, cudaSetDevice(m->device));
  for (uint32_t i = 0; i + 1 < n; i++)  // KV-fill-only steps: no output suffix (src/forward.rs:947-965)
    if (int st = step_no_suffix(m, tokens[i], pos_base + i)) return st;
  return bp_model_step_topk(m, tokens[n - 1], pos_base + n - 1, k, logits, indices);
}

int bp_model_prefill_topk(bp_model* m, const uint32_t* tokens, uint32_t n, uint32_t k, float* logits, uint32_t* indices) {
  if (int st = model_enter(m)) return st;
  if (!tokens || !logits || !indices) return mfail(m, BP_ERR_NULL, "null pointer argument");
  if (n == 0 || n > M_MAX) {
    char buf[160];
    snprintf(buf, sizeof buf, "prefill batch %u exceeds max_prefill_tokens %u", n, M_MAX);
    return mfail(m, BP_ERR_PREFILL_TOO_LARGE, buf, 0, n, M_MAX);
  }
  if (n > m->max_seq) {
    char buf[160];
    snprintf(buf, sizeof buf, "context overflow: pos %u + tokens %u > max_seq %u", 0u, n, m->max_seq);
    return mfail(m, BP_ERR_CONTEXT_OVERFLOW, buf, 0, n, m->max_seq);
  }
  for (uint32_t i = 0; i < n; i++)
    if (tokens[i] >= m->cfg.n_vocab) return mfail(m, BP_ERR_CONFIG, "invalid config: token id out of range");
  k = k < 1 ? 1 : (k > TOPK_MAX ? TOPK_MAX : k);
  const Config& c = m->cfg;
  cudaStream_t s = m->stream;
  const bool pdl = true;
  M_CUDA(m, cudaSetDevice(m->device));
  M_CUDA(m, cudaMemcpyAsync(m->tokens_dev, tokens, n * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
  M_CUDA(m, bp_q1_embed(pdl, s, m->embed, m->tokens_dev, n, m->x));
  for (uint32_t il = 0; il < c.n_layer; il++) {  // layer_step_matmul_in_pass, src/forward.rs:1075-1253
    const LayerTensors& lt = m->layers[il];
    uint32_t launches = 0;
    M_CUDA(m, bp_q1_rms_norm(pdl, s, m->x, m->x_norm, lt.attn_norm, c.n_embd, n, c.rms_eps));
    {
      const bp_q1_tensor w[3] = {lt.wq, lt.wk, lt.wv};
      __half* const out[3] = {m->q, m->k_cur, m->v_cur};
      if (int st = quantize_and_matmul(m, m->x_norm, c.n_embd, n, w, out, 3, false)) return st;
    }
    M_CUDA(m, bp_launch_q_norm_rope(m->attn, s, m->q, lt.q_norm, 0, n, &launches));
    M_CUDA(m, bp_launch_kv_writeback(m->attn, s, il, m->k_cur, m->v_cur, lt.k_norm, 0, n, &launches));
    M_CUDA(m, bp_launch_prefill(m->attn, s, il, m->q, m->attn_out, n, &launches));
    {
      __half* const out[1] = {m->x};
      if (int st = quantize_and_matmul(m, m->attn_out, c.q_dim, n, &lt.wo, out, 1, true)) return st;
    }
    M_CUDA(m, bp_q1_rms_norm(pdl, s, m->x, m->x_norm, lt.ffn_norm, c.n_embd, n, c.rms_eps));
    {
      const bp_q1_tensor w[2] = {lt.wg, lt.wu};
      __half* const out[2] = {m->gate, m->up};
      if (int st = quantize_and_matmul(m, m->x_norm, c.n_embd, n, w, out, 2, false)) return st;
    }
    M_CUDA(m, bp_q1_silu_mul(pdl, s, m->gate, m->up, m->ffn_in, static_cast<uint64_t>(n) * c.n_ff));
    {
      __half* const out[1] = {m->x};
      if (int st = quantize_and_matmul(m, m->ffn_in, c.n_ff, n, &lt.wd, out, 1, true)) return st;
    }
  }
  return output_suffix(m, n - 1, k, logits, indices);
}

int bp_model_read_hidden(bp_model* m, uint32_t row, void* x_host) {
  if (!m || !x_host) return BP_ERR_NULL;
  if (!m->x || row >= M_MAX) return mfail(m, BP_ERR_CONFIG, "invalid config: no such row");
  M_CUDA(m, cudaSetDevice(m->device));
  M_CUDA(m, cudaStreamSynchronize(m->stream));
  M_CUDA(m, cudaMemcpy(x_host, m->x + static_cast<size_t>(row) * m->cfg.n_embd, static_cast<size_t>(m->cfg.n_embd) * 2, cudaMemcpyDeviceToHost));
  return BP_OK;
}
int bp_model_read_logits(bp_model* m, void* logits_host) {
  if (!m || !logits_host) return BP_ERR_NULL;
  if (!m->logits) return mfail(m, BP_ERR_CONFIG, "invalid config: model is not loaded");
  M_CUDA(m, cudaSetDevice(m->device));
  M_CUDA(m, cudaStreamSynchronize(m->stream));
  M_CUDA(m, cudaMemcpy(logits_host, m->logits, static_cast<size_t>(m->cfg.n_vocab) * 2, cudaMemcpyDeviceToHost));
  return BP_OK;
}
int bp_model_attn_tap(bp_model* m, uint32_t mode, void* buf_host) {
  if (!m) return BP_ERR_NULL;
  if (mode > 2 || (mode != 0 && !buf_host)) return mfail(m, BP_ERR_CONFIG, "invalid config: tap mode is 0, 1 or 2 with a buffer");
  m->tap_mode = mode;
  m->tap_buf = static_cast<uint8_t*>(buf_host);
  return BP_OK;
}

// ---- sampler ----------------------------------------------------------------------------------------
void bp_sampler_default(bp_sampler* s) {
  if (!s) return;
  s->temperature = 1.0f;
  s->top_k = 0;
  s->top_p = -1.0f;
  s->seed = 0;
}
uint32_t bp_effective_k(const bp_sampler* s) { return s && s->top_k > 0 ? (s->top_k < TOPK_MAX ? s->top_k : TOPK_MAX) : TOPK_MAX; }

float bp_uniform_f32(uint64_t seed) {  // SplitMix64 finaliser, top 24 bits -> [0, 1)
  uint64_t z = seed + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return static_cast<float>(static_cast<uint32_t>(z >> 40)) / static_cast<float>(1u << 24);
}

uint32_t bp_sample_from_topk(const float* logits, const uint32_t* indices, uint32_t n, const bp_sampler* s, uint32_t pos) {
  if (n == 0 || !logits || !indices || !s) return 0;
  if (s->temperature <= 0.0f || s->top_k == 1) return indices[0];
  const uint32_t kk = s->top_k > 0 && s->top_k < n ? s->top_k : n;
  const float inv_t = 1.0f / s->temperature;
  const float max_l = logits[0] * inv_t;
  std::vector<float> probs(kk);
  float sum = 0.0f;
  for (uint32_t i = 0; i < kk; i++) {
    probs[i] = expf(fmaf(logits[i], inv_t, -max_l));
    sum += probs[i];
  }
  if (!(sum > 0.0f) || !isfinite(sum)) return indices[0];
  for (float& p : probs) p /= sum;
  const float cutoff = s->top_p < 0.0f ? 1.0f : (s->top_p > 1.0f ? 1.0f : s->top_p);
  float cum = 0.0f;
  uint32_t keep = kk;
  for (uint32_t i = 0; i < kk; i++) {
    cum += probs[i];
    if (cum >= cutoff) {
      keep = i + 1;
      break;
    }
  }
  float kept_sum = 0.0f;
  for (uint32_t i = 0; i < keep; i++) kept_sum += probs[i];
  if (!(kept_sum > 0.0f) || !isfinite(kept_sum)) return indices[0];
  const float r = bp_uniform_f32(s->seed + pos) * kept_sum;
  float acc = 0.0f;
  for (uint32_t i = 0; i < keep; i++) {
    acc += probs[i];
    if (r < acc) return indices[i];
  }
  return indices[keep - 1];
}

// ---- session ------------------------------------------------------------------------------------------
int bp_session_create(bp_model* m, bp_session** out) {
  if (!m || !out) return BP_ERR_NULL;
  *out = new (std::nothrow) bp_session{m, 0};
  return *out ? BP_OK : BP_ERR_CUDA;
}
void bp_session_free(bp_session* s) { delete s; }
uint32_t bp_session_pos(const bp_session* s) { return s ? s->pos : 0; }
void bp_session_reset(bp_session* s) {
  if (s) s->pos = 0;
}

static int overflow(bp_model* m, uint32_t pos, uint32_t n) {
  char buf[160];
  snprintf(buf, sizeof buf, "context overflow: pos %u + tokens %u > max_seq %u", pos, n, m->max_seq);
  return mfail(m, BP_ERR_CONTEXT_OVERFLOW, buf, pos, n, m->max_seq);
}

int bp_session_prefill(bp_session* s, const uint32_t* tokens, uint32_t n, const bp_sampler* sampler, uint32_t* chosen) {
  if (!s || !sampler || !chosen) return BP_ERR_NULL;
  bp_model* m = s->m;
  if (int st = model_enter(m)) return st;
  if (s->pos != 0)
    return mfail(m, BP_ERR_CONFIG, "invalid config: Session::prefill requires pos == 0; use prefill_one_at_a_time for incremental prefill");
  if (static_cast<uint64_t>(s->pos) + n > m->max_seq) return overflow(m, s->pos, n);
  float logits[TOPK_MAX];
  uint32_t idx[TOPK_MAX];
  const uint32_t k = bp_effective_k(sampler);
  if (int st = bp_model_prefill_topk(m, tokens, n, k, logits, idx)) return st;
  *chosen = bp_sample_from_topk(logits, idx, k, sampler, s->pos);
  s->pos += n;
  return BP_OK;
}

int bp_session_prefill_one_at_a_time(bp_session* s, const uint32_t* tokens, uint32_t n, const bp_sampler* sampler, uint32_t* chosen) {
  if (!s || !sampler || !chosen) return BP_ERR_NULL;
  bp_model* m = s->m;
  if (int st = model_enter(m)) return st;
  if (static_cast<uint64_t>(s->pos) + n > m->max_seq) return overflow(m, s->pos, n);
  float logits[TOPK_MAX];
  uint32_t idx[TOPK_MAX];
  const uint32_t k = bp_effective_k(sampler);
  if (int st = bp_model_prefill_loop_topk(m, tokens, n, s->pos, k, logits, idx)) return st;
  *chosen = bp_sample_from_topk(logits, idx, k, sampler, s->pos);
  s->pos += n;
  return BP_OK;
}

int bp_session_step(bp_session* s, uint32_t token, const bp_sampler* sampler, uint32_t* chosen) {
  if (!s || !sampler || !chosen) return BP_ERR_NULL;
  bp_model* m = s->m;
  if (int st = model_enter(m)) return st;
  if (static_cast<uint64_t>(s->pos) + 1 > m->max_seq) return overflow(m, s->pos, 1);
  float logits[TOPK_MAX];
  uint32_t idx[TOPK_MAX];
  const uint32_t k = bp_effective_k(sampler);
  if (int st = bp_model_step_topk(m, token, s->pos, k, logits, idx)) return st;
  *chosen = bp_sample_from_topk(logits, idx, k, sampler, s->pos);
  s->pos += 1;
  return BP_OK;
}

int bp_session_generate(bp_session* s, uint32_t first_token, uint32_t max_new_tokens, const bp_sampler* sampler, bp_stop_fn stop,
                        bp_token_fn on_token, void* user, uint32_t* out_tokens, uint32_t* n_out, int32_t* stop_reason) {
  if (!s || !sampler || !stop_reason) return BP_ERR_NULL;
  bp_model* m = s->m;
  if (n_out) *n_out = 0;
  if (int st = model_enter(m)) return st;
  *stop_reason = BP_STOP_MAX_TOKENS;
  if (max_new_tokens == 0) return BP_OK;
  if (static_cast<uint64_t>(s->pos) + 1 > m->max_seq) return overflow(m, s->pos, 1);
  const uint32_t k = bp_effective_k(sampler);
  uint32_t token = first_token, emitted = 0;
  for (uint32_t i = 0; i < max_new_tokens; i++) {
    float logits[TOPK_MAX];
    uint32_t idx[TOPK_MAX];
    if (static_cast<uint64_t>(s->pos) + 1 > m->max_seq) return overflow(m, s->pos, 1);
    if (int st = bp_model_step_topk(m, token, s->pos, k, logits, idx)) return st;
    const uint32_t chosen = bp_sample_from_topk(logits, idx, k, sampler, s->pos);
    s->pos += 1;
    const bool is_stop = stop ? stop(chosen, user) != 0 : chosen == m->cfg.eos_token_id;
    if (is_stop) {
      *stop_reason = BP_STOP_EOS;
      break;
    }
    if (on_token) on_token(chosen, user);
    if (out_tokens) out_tokens[emitted] = chosen;
    emitted++;
    token = chosen;
  }
  if (n_out) *n_out = emitted;
  return BP_OK;
}

uint64_t bp_session_snapshot_size(const bp_session* s) { return s ? bp_snapshot_size(s->m->attn, s->pos) : 0; }
int bp_session_snapshot(bp_session* s, void* blob, uint64_t blob_bytes) {
  if (!s) return BP_ERR_NULL;
  return attn_status(s->m, bp_snapshot_capture(s->m->attn, s->pos, blob, blob_bytes));
}
int bp_session_restore(bp_session* s, const void* blob, uint64_t blob_bytes) {
  if (!s) return BP_ERR_NULL;
  uint32_t pos = 0;
  const int st = attn_status(s->m, bp_snapshot_apply(s->m->attn, blob, blob_bytes, &pos));
  if (st == BP_OK) s->pos = pos;
  return st;
}

}  // extern "C"
