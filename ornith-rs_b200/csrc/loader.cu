// Artifact loader: config.json + safetensors shards -> orn_model.
//
// Follows src/safetensors.rs:189-308 (8-byte little-endian header length, JSON
// header, raw tensor bytes; shards listed by model.safetensors.index.json),
// src/weights.rs:41-279 (per-module quantisation from config.json, the
// three-tensor k-quant modules `.weight/.scales/.dm`, affine modules
// `.weight/.scales/.biases`, numbered MTP experts stacked at load) and
// src/model/config.rs:44-158 (text_config fields).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "orn_internal.h"

namespace {

// ---------------------------------------------------------------- tiny JSON
struct JVal {
  enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JVal> arr;
  std::vector<std::pair<std::string, JVal>> obj;
  const JVal* get(const std::string& k) const {
    if (type != Obj) return nullptr;
    for (auto& kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(const char* s) {
    size_t n = strlen(s);
    if ((size_t)(end - p) >= n && memcmp(p, s, n) == 0) { p += n; return true; }
    return false;
  }
  std::string string() {
    std::string out;
    if (p >= end || *p != '"') { ok = false; return out; }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {  // keep the escape verbatim; tensor names are ASCII
            out += "\\u";
            break;
          }
          default: out += *p; break;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  JVal value() {
    JVal v;
    ws();
    if (p >= end) { ok = false; return v; }
    if (*p == '{') {
      v.type = JVal::Obj;
      ++p; ws();
      if (p < end && *p == '}') { ++p; return v; }
      while (ok) {
        ws();
        std::string k = string();
        ws();
        if (p >= end || *p != ':') { ok = false; break; }
        ++p;
        JVal c = value();
        v.obj.emplace_back(std::move(k), std::move(c));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; break; }
        ok = false;
      }
    } else if (*p == '[') {
      v.type = JVal::Arr;
      ++p; ws();
      if (p < end && *p == ']') { ++p; return v; }
      while (ok) {
        v.arr.push_back(value());
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; break; }
        ok = false;
      }
    } else if (*p == '"') {
      v.type = JVal::Str;
      v.str = string();
    } else if (lit("true")) { v.type = JVal::Bool; v.b = true; }
    else if (lit("false")) { v.type = JVal::Bool; v.b = false; }
    else if (lit("null")) { v.type = JVal::Null; }
    else {
      // the header of a memory-mapped file is not NUL-terminated: parse from a bounded copy
      char tmp[64];
      size_t n = 0;
      while (p + n < end && n + 1 < sizeof tmp && (isdigit((unsigned char)p[n]) || strchr("+-.eE", p[n]) != nullptr)) {
        tmp[n] = p[n];
        ++n;
      }
      tmp[n] = 0;
      char* e = nullptr;
      v.type = JVal::Num;
      v.num = strtod(tmp, &e);
      if (e == tmp) ok = false;
      p += (e - tmp);
    }
    return v;
  }
};

bool parse_json(const char* data, size_t n, JVal* out) {
  JParser ps{data, data + n};
  *out = ps.value();
  return ps.ok;
}

bool read_file(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  fseek(f, 0, SEEK_END);
  long n = ftell(f);
  fseek(f, 0, SEEK_SET);
  out->resize((size_t)n);
  bool ok = n == 0 || fread(&(*out)[0], 1, (size_t)n, f) == (size_t)n;
  fclose(f);
  return ok;
}

// ---------------------------------------------------------------- safetensors
struct TInfo {
  std::string dtype;
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
};
struct Shard {
  void* map = nullptr;
  size_t size = 0;
};
struct Store {
  std::vector<Shard> shards;
  std::map<std::string, TInfo> tensors;
  ~Store() {
    for (auto& s : shards)
      if (s.map) munmap(s.map, s.size);
  }
};

bool open_shard(const std::string& path, Store* st, std::string* err) {
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) { *err = "cannot open " + path; return false; }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); *err = "short file " + path; return false; }
  void* mp = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (mp == MAP_FAILED) { *err = "mmap failed for " + path; return false; }
  st->shards.push_back(Shard{mp, (size_t)sb.st_size});
  const uint8_t* base = (const uint8_t*)mp;
  uint64_t hlen = 0;
  memcpy(&hlen, base, 8);
  if (hlen > (uint64_t)sb.st_size - 8) { *err = "bad header length in " + path; return false; }
  JVal hdr;
  if (!parse_json((const char*)base + 8, (size_t)hlen, &hdr) || hdr.type != JVal::Obj) {
    *err = "bad safetensors header in " + path;
    return false;
  }
  const uint8_t* data = base + 8 + hlen;
  const size_t data_size = (size_t)sb.st_size - 8 - (size_t)hlen;
  for (auto& kv : hdr.obj) {
    if (kv.first == "__metadata__") continue;
    const JVal* dt = kv.second.get("dtype");
    const JVal* sh = kv.second.get("shape");
    const JVal* off = kv.second.get("data_offsets");
    if (!dt || !sh || !off || off->arr.size() != 2) { *err = "bad tensor entry " + kv.first; return false; }
    TInfo ti;
    ti.dtype = dt->str;
    bool shape_ok = true;
    for (auto& d : sh->arr) {
      if (d.type != JVal::Num || d.num < 0 || d.num > 2147483647.0 || d.num != (double)(int64_t)d.num) shape_ok = false;
      ti.shape.push_back((int64_t)d.num);
    }
    if (!shape_ok) { *err = "bad shape for " + kv.first; return false; }
    size_t a = (size_t)off->arr[0].num, b = (size_t)off->arr[1].num;
    if (a > b || b > data_size) { *err = "tensor out of bounds: " + kv.first; return false; }
    ti.data = data + a;
    ti.nbytes = b - a;
    st->tensors[kv.first] = ti;
  }
  return true;
}

bool ends_with(const std::string& s, const std::string& suf) {
  return s.size() >= suf.size() && s.compare(s.size() - suf.size(), suf.size(), suf) == 0;
}

int64_t numel(const TInfo& t) {
  int64_t n = 1;
  for (auto d : t.shape) n *= d;
  return n;
}
// bytes the declared dtype and shape ask for must be the bytes the file holds for the tensor
bool bytes_match(const TInfo& t, size_t elem) { return !t.shape.empty() && numel(t) > 0 && (size_t)numel(t) * elem == t.nbytes; }

// per-module quantisation of config.json (src/weights.rs:41-98): a default {group_size, bits, mode}
// and overrides keyed by module path
struct QSpec {
  int group = 0, bits = 0;
  std::string mode;  // "affine", "q4k", "q6k", "nvfp4", ...
  bool present = false;
};

}  // namespace

extern "C" int32_t orn_model_load(orn_ctx* ctx, const char* dir_c, int32_t max_ctx, orn_model** out) {
  if (!ctx || !dir_c || !out) return ORN_ERR_ARG;
  *out = nullptr;
  const std::string dir(dir_c);
  // ---- config.json (src/model/config.rs:44-158)
  std::string raw;
  if (!read_file(dir + "/config.json", &raw)) ORN_FAIL(ctx, ORN_ERR_IO, "config.json: cannot read");
  JVal cfgj;
  if (!parse_json(raw.data(), raw.size(), &cfgj)) ORN_FAIL(ctx, ORN_ERR_IO, "config.json: parse error");
  const JVal* t = cfgj.get("text_config");
  if (!t) t = &cfgj;
  bool missing = false;
  std::string missing_key;
  auto u = [&](const char* k) -> int {
    const JVal* v = t->get(k);
    if (!v || v->type != JVal::Num) { if (!missing) missing_key = k; missing = true; return 0; }
    return (int)v->num;
  };
  auto f = [&](const char* k, float d) -> float {
    const JVal* v = t->get(k);
    return (v && v->type == JVal::Num) ? (float)v->num : d;
  };
  orn_config c{};
  c.hidden = u("hidden_size");
  c.n_layers = u("num_hidden_layers");
  c.n_heads = u("num_attention_heads");
  c.n_kv_heads = u("num_key_value_heads");
  { const JVal* v = t->get("head_dim"); c.head_dim = v ? (int)v->num : (c.n_heads ? c.hidden / c.n_heads : 0); }
  { const JVal* v = t->get("full_attention_interval"); c.full_attn_interval = v ? (int)v->num : 4; }
  const JVal* rope = t->get("rope_parameters");
  float theta = f("rope_theta", 100000.0f), prf = f("partial_rotary_factor", 0.25f);
  if (rope) {
    if (const JVal* v = rope->get("rope_theta")) theta = (float)v->num;
    if (const JVal* v = rope->get("partial_rotary_factor")) prf = (float)v->num;
  }
  c.rope_theta = theta;
  c.rope_dims = (int)((float)c.head_dim * prf);
  c.gdn_k_heads = u("linear_num_key_heads");
  c.gdn_v_heads = u("linear_num_value_heads");
  c.gdn_head_dim = u("linear_key_head_dim");
  c.gdn_conv_kernel = u("linear_conv_kernel_dim");
  c.n_experts = u("num_experts");
  c.top_k = u("num_experts_per_tok");
  c.expert_inter = u("moe_intermediate_size");
  c.shared_inter = u("shared_expert_intermediate_size");
  { const JVal* v = t->get("norm_topk_prob"); c.norm_topk_prob = (!v || v->type != JVal::Bool) ? 1 : (v->b ? 1 : 0); }
  c.vocab = u("vocab_size");
  c.rms_eps = f("rms_norm_eps", 1e-6f);
  c.max_ctx = max_ctx;
  if (missing) ORN_FAIL(ctx, ORN_ERR_IO, "config.json: missing " + missing_key);
  if (u("linear_value_head_dim") != c.gdn_head_dim) ORN_FAIL(ctx, ORN_ERR_ARG, "config.json: key and value head dims differ");

  // ---- quantization block (src/weights.rs:49-79); absent in hand-made artifacts: formats then follow the tensors
  QSpec qdef;
  std::map<std::string, QSpec> qmods;
  if (const JVal* q = cfgj.get("quantization")) {
    if (q->type != JVal::Obj) ORN_FAIL(ctx, ORN_ERR_IO, "config.json: quantization is not an object");
    const JVal* g = q->get("group_size");
    const JVal* b = q->get("bits");
    if (!g || !b || g->type != JVal::Num || b->type != JVal::Num) ORN_FAIL(ctx, ORN_ERR_IO, "config.json: quantization.group_size / bits");
    qdef.group = (int)g->num; qdef.bits = (int)b->num; qdef.present = true;
    const JVal* md = q->get("mode");
    qdef.mode = (md && md->type == JVal::Str) ? md->str : "affine";  // older artifacts carry no mode (weights.rs:52-53)
    for (auto& kv : q->obj) {
      if (kv.second.type != JVal::Obj) continue;
      QSpec sp = qdef;
      if (const JVal* v = kv.second.get("group_size")) sp.group = (int)v->num;
      if (const JVal* v = kv.second.get("bits")) sp.bits = (int)v->num;
      if (const JVal* v = kv.second.get("mode")) if (v->type == JVal::Str) sp.mode = v->str;
      qmods[kv.first] = sp;
    }
  }
  auto spec_of = [&](const std::string& mod) -> QSpec {
    auto it = qmods.find(mod);
    return it == qmods.end() ? qdef : it->second;
  };

  // ---- shards (src/safetensors.rs:296-308) and the MTP sidecar (mtp.rs:270-279)
  Store st;
  std::string err;
  std::vector<std::string> files;
  std::string idx;
  if (read_file(dir + "/model.safetensors.index.json", &idx)) {
    JVal ij;
    if (!parse_json(idx.data(), idx.size(), &ij)) ORN_FAIL(ctx, ORN_ERR_IO, "model.safetensors.index.json: parse error");
    const JVal* wm = ij.get("weight_map");
    if (!wm || wm->type != JVal::Obj) ORN_FAIL(ctx, ORN_ERR_IO, "index has no weight_map");
    for (auto& kv : wm->obj) {
      bool seen = false;
      for (auto& fnm : files) seen = seen || fnm == kv.second.str;
      if (!seen) files.push_back(kv.second.str);
    }
  } else {
    files.push_back("model.safetensors");
  }
  for (auto& fnm : files)
    if (!open_shard(dir + "/" + fnm, &st, &err)) ORN_FAIL(ctx, ORN_ERR_IO, err);
  {
    std::string rel = "mtp/weights.safetensors";
    if (const JVal* x = cfgj.get("mlx_lm_extra_tensors"))
      if (const JVal* mf = x->get("mtp_file")) rel = mf->str;
    struct stat sb;
    if (stat((dir + "/" + rel).c_str(), &sb) == 0)
      if (!open_shard(dir + "/" + rel, &st, &err)) ORN_FAIL(ctx, ORN_ERR_IO, err);
  }

  orn_model* m = nullptr;
  int rc = orn_model_create(ctx, &c, &m);
  if (rc != ORN_OK) return rc;
  auto fail = [&](int code, const std::string& msg) {
    orn_model_destroy(m);
    ctx->err = msg;
    return code;
  };

  // ---- classify and upload
  const std::string mtp_moe = "mtp.layers.0.mlp.";
  const std::string mtp_exp = "mtp.layers.0.mlp.experts.";
  std::map<std::string, bool> stacked_done;
  for (auto& kv : st.tensors) {
    const std::string& name = kv.first;
    const TInfo& ti = kv.second;
    if (ends_with(name, ".scales") || ends_with(name, ".biases") || ends_with(name, ".dm")) continue;
    if (name.find("visual") != std::string::npos || name.find("vision") != std::string::npos) continue;
    // numbered MTP experts: stack 0..E-1 into one [E, O, K] bf16 matrix (weights.rs:237-279)
    if (name.rfind(mtp_exp, 0) == 0) {
      size_t dot = name.find('.', mtp_exp.size());
      if (dot == std::string::npos) continue;
      std::string proj = name.substr(dot + 1);  // gate_proj.weight
      if (stacked_done[proj]) continue;
      stacked_done[proj] = true;
      if (ti.dtype != "BF16" || ti.shape.size() != 2 || !bytes_match(ti, 2))
        return fail(ORN_ERR_ARG, "mtp expert tensor is not 2-D bf16 of its declared size: " + name);
      const int O = (int)ti.shape[0], K = (int)ti.shape[1];
      std::vector<uint8_t> buf((size_t)c.n_experts * O * K * 2);
      for (int e = 0; e < c.n_experts; ++e) {
        auto it = st.tensors.find(mtp_exp + std::to_string(e) + "." + proj);
        if (it == st.tensors.end() || it->second.nbytes != (size_t)O * K * 2)
          return fail(ORN_ERR_IO, "missing MTP expert " + std::to_string(e) + " " + proj);
        memcpy(buf.data() + (size_t)e * O * K * 2, it->second.data, (size_t)O * K * 2);
      }
      orn_linear* L = nullptr;
      rc = orn_linear_create(ctx, ORN_BF16, c.n_experts, O, K, buf.data(), nullptr, nullptr, &L);
      if (rc != ORN_OK) { orn_model_destroy(m); return rc; }
      std::string mod = proj.substr(0, proj.size() - strlen(".weight"));
      orn_model_set_linear(m, (mtp_moe + "switch_mlp." + mod).c_str(), L);
      continue;
    }
    if (ends_with(name, ".weight")) {
      const std::string mod = name.substr(0, name.size() - strlen(".weight"));
      auto sc = st.tensors.find(mod + ".scales");
      if (sc != st.tensors.end()) {
        auto dmq = st.tensors.find(mod + ".dm");
        auto bia = st.tensors.find(mod + ".biases");
        int kind;
        const TInfo* third;
        // leading expert axis, then [O, packed K]
        if (ti.shape.size() < 2 || sc->second.shape.empty()) return fail(ORN_ERR_ARG, "quantised weight is not a matrix: " + name);
        const int E = ti.shape.size() == 3 ? (int)ti.shape[0] : 1;
        const int O = (int)ti.shape[ti.shape.size() - 2];
        const int64_t packed = ti.shape.back();  // u32 words per row
        const int64_t scols = sc->second.shape.back();
        if (packed <= 0 || scols <= 0 || O <= 0 || E <= 0) return fail(ORN_ERR_ARG, "empty quantised tensor: " + mod);
        const QSpec sp = spec_of(mod);
        int K;
        const bool as_kquant = sp.present ? (sp.mode == "q4k" || sp.mode == "q6k") : dmq != st.tensors.end();
        if (sp.present && sp.mode != "affine" && !as_kquant)
          return fail(ORN_ERR_ARG, "quantization mode '" + sp.mode + "' is not on this path: " + mod);
        if (as_kquant) {
          // kquant_matrix (src/weights.rs:199-227): .weight/.scales/.dm, never .biases, super-blocks of 256
          if (dmq == st.tensors.end() || bia != st.tensors.end())
            return fail(ORN_ERR_ARG, "k-quant module must carry .dm and no .biases: " + mod);
          if (sp.present && sp.group != 256) return fail(ORN_ERR_ARG, "k-quant group_size must be 256: " + mod);
          third = &dmq->second;
          if (third->shape.empty()) return fail(ORN_ERR_ARG, "k-quant .dm has no shape: " + mod);
          const int64_t last = third->shape.back();
          const bool q4 = sp.present ? sp.mode == "q4k" : last == 2;
          if (q4 && last == 2) { kind = ORN_Q4K; K = (int)(packed * 8); }
          else if (!q4 && last == 1) { kind = ORN_Q6K; K = (int)(packed * 16 / 3); }
          else return fail(ORN_ERR_ARG, "k-quant .dm width does not match the module's mode: " + mod);
        } else {
          // quant_matrix (src/weights.rs:132-172): mlx affine, bits and group size from config.json
          if (bia == st.tensors.end() || dmq != st.tensors.end())
            return fail(ORN_ERR_ARG, "affine module must carry .biases and no .dm: " + mod);
          third = &bia->second;
          int bits = sp.bits, group = sp.group;
          if (!sp.present) {  // no quantization block: the 8-bit group-64 layout is the only one that can be assumed
            bits = 8; group = 64;
          }
          if (bits == 8 && group == 64) kind = ORN_A8;
          else if (bits == 4 && group == 32) kind = ORN_A4;
          else return fail(ORN_ERR_ARG, "affine module is neither 8-bit group-64 nor 4-bit group-32 (unsupported on this path): " + mod);
          K = (int)(packed * 32 / bits);
          if (scols * group != K) return fail(ORN_ERR_ARG, "affine module's scales do not match its bits and group size: " + mod);
        }
        size_t aw, as, ab;
        linear_artifact_sizes(kind, E, O, K, &aw, &as, &ab);
        if (ti.nbytes != aw || sc->second.nbytes != as || third->nbytes != ab)
          return fail(ORN_ERR_ARG, "tensor sizes do not match the declared shapes: " + mod);
        orn_linear* L = nullptr;
        rc = orn_linear_create(ctx, kind, E, O, K, ti.data, sc->second.data, third->data, &L);
        if (rc != ORN_OK) { orn_model_destroy(m); return rc; }
        orn_model_set_linear(m, mod.c_str(), L);
        continue;
      }
      if (ti.dtype == "BF16" && ti.shape.size() == 2) {
        if (!bytes_match(ti, 2)) return fail(ORN_ERR_ARG, "tensor bytes do not match its shape: " + name);
        orn_linear* L = nullptr;
        rc = orn_linear_create(ctx, ORN_BF16, 1, (int)ti.shape[0], (int)ti.shape[1], ti.data, nullptr, nullptr, &L);
        if (rc != ORN_OK) { orn_model_destroy(m); return rc; }
        // the MTP head's MoE matrices are addressed by module name
        std::string reg = (name.rfind(mtp_moe, 0) == 0) ? mod : name;
        orn_model_set_linear(m, reg.c_str(), L);
        continue;
      }
    }
    if (ti.dtype == "BF16") {
      if (!bytes_match(ti, 2)) return fail(ORN_ERR_ARG, "tensor bytes do not match its shape: " + name);
      rc = orn_model_set_tensor(m, name.c_str(), (const uint16_t*)ti.data, (size_t)numel(ti));
      if (rc != ORN_OK) { orn_model_destroy(m); return rc; }
    }
    // other dtypes (e.g. vision tensors in float) are not on this path
  }
  *out = m;
  return ORN_OK;
}
