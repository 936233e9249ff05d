// Model directory loader (host C++): the counterpart of spbitnet::Model::load (src/model.cu:179-311).
//
//   <dir>/config.json     architecture (src/model.cu:72-90; defaults: rms_norm_eps 1e-5, rope_theta 1e4,
//                         head_dim = hidden / heads, bos 128000, eos 128001)
//   <dir>/manifest.json   {"weights": {name: entry}}: sparse_ternary entries (meta_file, values_file, shape,
//                         meta_stride, values_stride, gamma), dense entries (file, dtype, shape), {"dtype":"tied"}
//   <dir>/weights/...     raw little-endian arrays
// Differences from the reference loader, none visible in the results: one pooled device allocation instead of one
// cudaMalloc per tensor (about 550 for the 2B-4T model), files streamed through one pinned staging buffer,
// sizes checked against shape and strides before anything is uploaded, and every sparse tensor's bitmaps
// validated (exactly two bits per group) because the kernels assume it.  Errors come back as a status and a
// message instead of an exception.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/spbitnet_b200.h"
#include "json_min.h"

namespace spb {
int fail(int code, const char* fmt, ...);
}

struct spb_model {
    spb_model_config cfg{};
    int bos_token_id = 128000, eos_token_id = 128001;
    bool tied = true;
    uint8_t* pool = nullptr;
    size_t pool_bytes = 0;
    struct Sparse { size_t meta_off, values_off; float gamma; int rows, cols, ms, vs; };
    std::vector<Sparse> linear;       // layers x 7
    std::vector<long long> norm_off;  // layers x 4, -1 when absent
    size_t embed_off = 0, lm_head_off = 0, final_norm_off = 0;
    int device = 0;
};

namespace {

const char* kLinearNames[7] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                               "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"};
const char* kNormNames[4] = {"input_layernorm", "post_attention_layernorm", "self_attn.attn_sub_norm", "mlp.ffn_sub_norm"};

bool read_text(const std::string& path, std::string* out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    std::stringstream buf;
    buf << f.rdbuf();
    *out = buf.str();
    return true;
}

long long file_size(const std::string& path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    return f ? static_cast<long long>(f.tellg()) : -1;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Piece {  // one file -> one place in the pool
    std::string path;
    size_t offset, bytes;
    bool bitmaps;  // validate as sparse metadata
    int rows, cols, ms;
};

}  // namespace

extern "C" spb_model* spb_model_load(const char* model_dir) {
    using spb::json::Value;
    if (!model_dir) {
        spb::fail(SPB_E_INVALID, "spb_model_load: null path");
        return nullptr;
    }
    const std::string root(model_dir);
    std::string text;
    Value cfgj, man;
    try {
        if (!read_text(root + "/config.json", &text)) throw std::runtime_error("cannot open config.json");
        cfgj = spb::json::parse(text);
        if (!read_text(root + "/manifest.json", &text)) throw std::runtime_error("cannot open manifest.json");
        man = spb::json::parse(text);
    } catch (const std::exception& e) {
        spb::fail(SPB_E_FORMAT, "spb_model_load: %s: %s", model_dir, e.what());
        return nullptr;
    }
    auto geti = [&](const char* k, long long d) { const Value* v = cfgj.find(k); return v ? v->as_int(d) : d; };
    auto getd = [&](const char* k, double d) { const Value* v = cfgj.find(k); return v ? v->as_double(d) : d; };
    auto* m = new spb_model();
    spb_model_config& c = m->cfg;
    c.hidden_size = static_cast<int>(geti("hidden_size", 0));
    c.num_hidden_layers = static_cast<int>(geti("num_hidden_layers", 0));
    c.num_attention_heads = static_cast<int>(geti("num_attention_heads", 0));
    c.num_key_value_heads = static_cast<int>(geti("num_key_value_heads", c.num_attention_heads));
    c.intermediate_size = static_cast<int>(geti("intermediate_size", 0));
    c.vocab_size = static_cast<int>(geti("vocab_size", 0));
    c.max_position_embeddings = static_cast<int>(geti("max_position_embeddings", 4096));
    c.head_dim = static_cast<int>(geti("head_dim", c.num_attention_heads > 0 ? c.hidden_size / c.num_attention_heads : 0));
    c.rms_norm_eps = static_cast<float>(getd("rms_norm_eps", 1e-5));
    c.rope_theta = static_cast<float>(getd("rope_theta", 10000.0));
    m->bos_token_id = static_cast<int>(geti("bos_token_id", 128000));
    m->eos_token_id = static_cast<int>(geti("eos_token_id", 128001));
    auto bail = [&](int code, const std::string& msg) -> spb_model* {
        spb::fail(code, "spb_model_load: %s", msg.c_str());
        if (m->pool) cudaFree(m->pool);
        delete m;
        return nullptr;
    };
    if (c.hidden_size <= 0 || c.num_hidden_layers < 0 || c.num_attention_heads <= 0 || c.num_key_value_heads <= 0 ||
        c.intermediate_size <= 0 || c.vocab_size <= 0 || c.head_dim <= 0)
        return bail(SPB_E_FORMAT, "config.json: missing or non-positive architecture field");
    const Value* weights = man.find("weights");
    if (!weights || !weights->is(Value::Object)) return bail(SPB_E_FORMAT, "manifest.json: no \"weights\" object");

    // ---- plan: every file's place in one pool, sizes checked against the manifest and the files ----
    std::vector<Piece> pieces;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off = align_up(off + bytes, 256); return o; };
    std::string err;
    auto dense = [&](const std::string& name, const char* dtype, size_t elem, size_t count, size_t* where) -> bool {
        const Value* e = weights->find(name);
        if (!e) { err = "manifest.json: no entry " + name; return false; }
        const Value* dt = e->find("dtype");
        const Value* file = e->find("file");
        if (!dt || dt->str != dtype || !file) { err = name + ": expected a " + dtype + " tensor with a file"; return false; }
        const std::string path = root + "/" + file->str;
        if (file_size(path) != static_cast<long long>(elem * count)) {
            err = name + ": " + file->str + " does not hold " + std::to_string(elem * count) + " bytes";
            return false;
        }
        *where = take(elem * count);
        pieces.push_back(Piece{path, *where, elem * count, false, 0, 0, 0});
        return true;
    };
    const size_t H = static_cast<size_t>(c.hidden_size), V = static_cast<size_t>(c.vocab_size);
    if (!dense("embed_tokens", "float16", 2, V * H, &m->embed_off)) return bail(SPB_E_FORMAT, err);
    if (!dense("norm", "float32", 4, H, &m->final_norm_off)) return bail(SPB_E_FORMAT, err);
    {
        const Value* head = weights->find("lm_head");
        const Value* dt = head ? head->find("dtype") : nullptr;
        m->tied = !head || (dt && dt->str == "tied");
        if (!m->tied && !dense("lm_head", "float16", 2, V * H, &m->lm_head_off)) return bail(SPB_E_FORMAT, err);
    }
    const int qdim = c.num_attention_heads * c.head_dim, kvdim = c.num_key_value_heads * c.head_dim;
    const int want_rows[7] = {qdim, kvdim, kvdim, c.hidden_size, c.intermediate_size, c.intermediate_size, c.hidden_size};
    const int want_cols[7] = {c.hidden_size, c.hidden_size, c.hidden_size, qdim, c.hidden_size, c.hidden_size, c.intermediate_size};
    for (int l = 0; l < c.num_hidden_layers; ++l) {
        for (int i = 0; i < 7; ++i) {
            const std::string name = "layers." + std::to_string(l) + "." + kLinearNames[i];
            const Value* e = weights->find(name);
            if (!e) return bail(SPB_E_FORMAT, "manifest.json: no entry " + name);
            const Value *dt = e->find("dtype"), *shape = e->find("shape"), *mf = e->find("meta_file"), *vf = e->find("values_file");
            const Value *msv = e->find("meta_stride"), *vsv = e->find("values_stride"), *gm = e->find("gamma");
            if (!dt || dt->str != "sparse_ternary" || !shape || shape->items.size() != 2 || !mf || !vf || !msv || !vsv || !gm)
                return bail(SPB_E_FORMAT, name + ": not a complete sparse_ternary entry");
            spb_model::Sparse s{};
            s.rows = static_cast<int>(shape->items[0].as_int());
            s.cols = static_cast<int>(shape->items[1].as_int());
            s.ms = static_cast<int>(msv->as_int());
            s.vs = static_cast<int>(vsv->as_int());
            s.gamma = static_cast<float>(gm->as_double());
            if (s.rows != want_rows[i] || s.cols != want_cols[i])
                return bail(SPB_E_FORMAT, name + ": shape does not match config.json");
            if (s.cols % 4 || s.ms < (s.cols / 4 + 7) / 8 || s.vs < (s.cols / 4 + 15) / 16)
                return bail(SPB_E_FORMAT, name + ": strides shorter than a row");
            const size_t mb = static_cast<size_t>(s.rows) * s.ms * 4, vb = static_cast<size_t>(s.rows) * s.vs * 4;
            const std::string mp = root + "/" + mf->str, vp = root + "/" + vf->str;
            if (file_size(mp) != static_cast<long long>(mb) || file_size(vp) != static_cast<long long>(vb))
                return bail(SPB_E_FORMAT, name + ": file sizes do not match shape and strides");
            s.meta_off = take(mb);
            pieces.push_back(Piece{mp, s.meta_off, mb, true, s.rows, s.cols, s.ms});
            s.values_off = take(vb);
            pieces.push_back(Piece{vp, s.values_off, vb, false, 0, 0, 0});
            m->linear.push_back(s);
        }
        for (int i = 0; i < 4; ++i) {
            const std::string name = "layers." + std::to_string(l) + "." + kNormNames[i];
            const size_t n = i == 3 ? static_cast<size_t>(c.intermediate_size) : H;
            size_t where = 0;
            if (weights->find(name)) {
                if (!dense(name, "float32", 4, n, &where)) return bail(SPB_E_FORMAT, err);
                m->norm_off.push_back(static_cast<long long>(where));
            } else if (i < 2) {
                return bail(SPB_E_FORMAT, "manifest.json: no entry " + name);
            } else {
                m->norm_off.push_back(-1);
            }
        }
    }
    // ---- upload: one pool, files streamed through a pinned staging buffer ----
    cudaGetDevice(&m->device);
    m->pool_bytes = off;
    if (cudaMalloc(&m->pool, m->pool_bytes) != cudaSuccess) {
        cudaGetLastError();
        return bail(SPB_E_CUDA, "cudaMalloc of " + std::to_string(m->pool_bytes) + " bytes failed");
    }
    const size_t kStage = 64u << 20;
    uint8_t* stage = nullptr;
    if (cudaMallocHost(&stage, kStage) != cudaSuccess) {
        cudaGetLastError();
        return bail(SPB_E_CUDA, "cudaMallocHost failed");
    }
    for (const Piece& p : pieces) {
        std::ifstream f(p.path, std::ios::binary);
        size_t done = 0;
        int row_in = 0;  // rows of bitmaps validated so far
        while (done < p.bytes) {
            size_t chunk = std::min(kStage, p.bytes - done);
            if (p.bitmaps) chunk = std::max<size_t>(1, chunk / (static_cast<size_t>(p.ms) * 4)) * p.ms * 4, chunk = std::min(chunk, p.bytes - done);
            f.read(reinterpret_cast<char*>(stage), static_cast<std::streamsize>(chunk));
            if (static_cast<size_t>(f.gcount()) != chunk) {
                cudaFreeHost(stage);
                return bail(SPB_E_FORMAT, p.path + ": short read");
            }
            if (p.bitmaps) {
                const int nrows = static_cast<int>(chunk / (static_cast<size_t>(p.ms) * 4));
                if (spb_validate_packed(reinterpret_cast<const uint32_t*>(stage), nrows, p.cols, p.ms) != SPB_OK) {
                    cudaFreeHost(stage);
                    return bail(SPB_E_FORMAT, p.path + ": a bitmap near row " + std::to_string(row_in) + " does not have exactly two bits");
                }
                row_in += nrows;
            }
            if (cudaMemcpy(m->pool + p.offset + done, stage, chunk, cudaMemcpyHostToDevice) != cudaSuccess) {
                cudaGetLastError();
                cudaFreeHost(stage);
                return bail(SPB_E_CUDA, "upload of " + p.path + " failed");
            }
            done += chunk;
        }
    }
    cudaFreeHost(stage);
    return m;
}

extern "C" void spb_model_destroy(spb_model* m) {
    if (!m) return;
    if (m->pool) cudaFree(m->pool);
    delete m;
}

extern "C" int spb_model_get_config(const spb_model* m, spb_model_config* cfg, int* bos_token_id, int* eos_token_id) {
    if (!m || !cfg) return spb::fail(SPB_E_INVALID, "spb_model_get_config: null pointer");
    *cfg = m->cfg;
    if (bos_token_id) *bos_token_id = m->bos_token_id;
    if (eos_token_id) *eos_token_id = m->eos_token_id;
    return SPB_OK;
}

extern "C" size_t spb_model_device_bytes(const spb_model* m) { return m ? m->pool_bytes : 0; }

extern "C" int spb_model_attach(const spb_model* m, spb_engine* e) {
    if (!m || !e) return spb::fail(SPB_E_INVALID, "spb_model_attach: null pointer");
    const uint8_t* p = m->pool;
    for (int l = 0; l < m->cfg.num_hidden_layers; ++l) {
        for (int i = 0; i < 7; ++i) {
            const spb_model::Sparse& s = m->linear[static_cast<size_t>(l) * 7 + i];
            const int rc = spb_engine_set_linear(e, l, i, reinterpret_cast<const uint32_t*>(p + s.meta_off),
                                                 reinterpret_cast<const uint32_t*>(p + s.values_off), s.gamma, s.rows, s.cols, s.ms, s.vs);
            if (rc) return rc;
        }
        for (int i = 0; i < 4; ++i) {
            const long long o = m->norm_off[static_cast<size_t>(l) * 4 + i];
            if (o >= 0)
                if (int rc = spb_engine_set_norm(e, l, i, reinterpret_cast<const float*>(p + o))) return rc;
        }
    }
    return spb_engine_set_globals(e, p + m->embed_off, m->tied ? nullptr : p + m->lm_head_off,
                                  reinterpret_cast<const float*>(p + m->final_norm_off));
}
