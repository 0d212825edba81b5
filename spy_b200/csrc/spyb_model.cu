// Whole-model path: GGUF -> device-resident quantized planes (optionally one tensor-parallel shard),
// and the LLaMa step executed as a fixed plan of fused kernels, replayed from a CUDA graph for
// single-token decode.
//
// The plan is the graph LLAMAModel::build_graph emits (model/src/llm/model/llama.cpp:123-222,
// plugin/attention.cpp:267-302, plugin/ffn.cpp:5-42, plugin/inout.cpp:5-78) with neighbouring
// operators folded into five kernels per layer:
//   1  NormRMS + Mul(attn_norm) + Q8_0 quantize -> Wq|Wk|Wv mat-vec -> RoPE(Q,K) + f16 KV append
//   2  attention (scores, masked softmax, PV)
//   3  Q8_0 quantize -> Wo mat-vec -> + residual
//   4  NormRMS + Mul(ffn_norm) + quantize -> Wup & Wgate mat-vec -> up * silu(gate)
//   5  Q8_0 quantize -> Wdown mat-vec -> + residual
// then NormRMS + Mul(output_norm) + quantize -> output mat-vec -> logits, and a greedy argmax that
// also gathers the next token's embedding.

#include <cmath>
#include <cstring>
#include <dlfcn.h>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "spyb_internal.h"

namespace spyb {

// ------------------------------------------------------------------------------------------ GGUF
// Same file layout GGUFAdapter::init_from_file reads (storage/src/adapter/gguf_adapter.cpp:90-190).
struct GgufTensor { int n_dim = 0; int64_t ne[4] = {1, 1, 1, 1}; int type = 0; uint64_t offset = 0; };

struct GgufFile {
    int      fd = -1;
    uint8_t *map = nullptr;
    size_t   size = 0;
    size_t   data_off = 0;
    std::map<std::string, GgufTensor> tensors;
    std::map<std::string, double>     num;    // numeric metadata
    std::map<std::string, std::string> str;
    int64_t  n_tokens = 0;

    ~GgufFile() { if (map) { munmap(map, size); } if (fd >= 0) { close(fd); } }

    bool open(const char *path, std::string *err) {
        fd = ::open(path, O_RDONLY);
        if (fd < 0) { *err = std::string("cannot open ") + path; return false; }
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size < 24) { *err = "file too small for a GGUF header"; return false; }
        size = (size_t)st.st_size;
        map = static_cast<uint8_t *>(mmap(nullptr, size, PROT_READ, MAP_SHARED, fd, 0));
        if (map == MAP_FAILED) { map = nullptr; *err = "mmap failed"; return false; }
        size_t pos = 0;
        auto need = [&](size_t n) { return pos + n <= size; };
        auto rd = [&](void *dst, size_t n) { if (!need(n)) { return false; } std::memcpy(dst, map + pos, n); pos += n; return true; };
        auto rd_str = [&](std::string *s) { uint64_t n; if (!rd(&n, 8) || !need(n)) { return false; } s->assign(reinterpret_cast<char *>(map + pos), n); pos += n; return true; };
        char magic[4]; uint32_t version; uint64_t n_tensors, n_kv;
        if (!rd(magic, 4) || std::memcmp(magic, "GGUF", 4) != 0) { *err = "bad GGUF magic"; return false; }
        if (!rd(&version, 4) || !rd(&n_tensors, 8) || !rd(&n_kv, 8)) { *err = "truncated GGUF header"; return false; }
        if (version != 3) { *err = "unsupported GGUF version"; return false; }
        static const int scalar_size[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
        auto rd_scalar = [&](uint32_t type, double *out) {
            uint8_t buf[8] = {0};
            if (type > 12 || scalar_size[type] == 0 || !rd(buf, scalar_size[type])) { return false; }
            switch (type) {
            case 0: *out = buf[0]; break; case 1: *out = (int8_t)buf[0]; break;
            case 2: { uint16_t v; std::memcpy(&v, buf, 2); *out = v; } break; case 3: { int16_t v; std::memcpy(&v, buf, 2); *out = v; } break;
            case 4: { uint32_t v; std::memcpy(&v, buf, 4); *out = v; } break; case 5: { int32_t v; std::memcpy(&v, buf, 4); *out = v; } break;
            case 6: { float v; std::memcpy(&v, buf, 4); *out = v; } break; case 7: *out = buf[0] != 0; break;
            case 10: { uint64_t v; std::memcpy(&v, buf, 8); *out = (double)v; } break; case 11: { int64_t v; std::memcpy(&v, buf, 8); *out = (double)v; } break;
            case 12: { double v; std::memcpy(&v, buf, 8); *out = v; } break;
            default: return false;
            }
            return true;
        };
        for (uint64_t i = 0; i < n_kv; ++i) {
            std::string key; uint32_t type;
            if (!rd_str(&key) || !rd(&type, 4)) { *err = "truncated GGUF metadata"; return false; }
            if (type == 8) { std::string v; if (!rd_str(&v)) { *err = "truncated GGUF string"; return false; } str[key] = v; }
            else if (type == 9) {
                uint32_t et; uint64_t n;
                if (!rd(&et, 4) || !rd(&n, 8)) { *err = "truncated GGUF array"; return false; }
                if (key == "tokenizer.ggml.tokens") { n_tokens = (int64_t)n; }
                for (uint64_t j = 0; j < n; ++j) {
                    if (et == 8) { std::string v; if (!rd_str(&v)) { *err = "truncated GGUF array"; return false; } }
                    else { double v; if (!rd_scalar(et, &v)) { *err = "bad GGUF array element"; return false; } }
                }
            } else { double v; if (!rd_scalar(type, &v)) { *err = "bad GGUF value type"; return false; } num[key] = v; }
        }
        for (uint64_t i = 0; i < n_tensors; ++i) {
            std::string name; GgufTensor t; uint32_t nd, ty;
            if (!rd_str(&name) || !rd(&nd, 4) || nd > 4) { *err = "truncated GGUF tensor info"; return false; }
            t.n_dim = (int)nd;
            for (uint32_t k = 0; k < nd; ++k) { uint64_t e; if (!rd(&e, 8)) { *err = "truncated GGUF tensor info"; return false; } t.ne[k] = (int64_t)e; }
            if (!rd(&ty, 4) || !rd(&t.offset, 8)) { *err = "truncated GGUF tensor info"; return false; }
            t.type = (int)ty;
            tensors[name] = t;
        }
        const size_t align = num.count("general.alignment") ? (size_t)num["general.alignment"] : 32;
        data_off = (pos + align - 1) / align * align;
        return true;
    }

    static int64_t row_bytes(int type, int64_t k) {
        switch (type) { case 0: return k * 4; case 1: return k * 2; case 2: return k / 32 * 18; case 8: return k / 32 * 34;
                        case 12: return k / 256 * 144; case 14: return k / 256 * 210; default: return -1; }
    }
    const uint8_t *data(const GgufTensor &t, std::string *err) const {
        const int64_t rb = row_bytes(t.type, t.ne[0]);
        if (rb < 0) { *err = "tensor type not supported"; return nullptr; }
        const size_t bytes = (size_t)rb * t.ne[1] * t.ne[2] * t.ne[3];
        if (data_off + t.offset + bytes > size) { *err = "tensor data runs past the end of the file"; return nullptr; }
        return map + data_off + t.offset;
    }
};

// ------------------------------------------------------------------------------------------ NCCL (loaded on demand)
struct NcclApi {
    struct Uid { char b[128]; };   // ncclUniqueId, passed by value
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, Uid, int) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool load() {
        if (lib) { return true; }
        lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) { return false; }
        GetUniqueId  = reinterpret_cast<decltype(GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
        CommInitRank = reinterpret_cast<decltype(CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
        AllGather    = reinterpret_cast<decltype(AllGather)>(dlsym(lib, "ncclAllGather"));
        CommDestroy  = reinterpret_cast<decltype(CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
        GetErrorString = reinterpret_cast<decltype(GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
        return GetUniqueId && CommInitRank && AllGather && CommDestroy;
    }
};
static NcclApi g_nccl;

constexpr int TMAX_COLUMNS = 8;        // activation columns the mat-vec passes hold
constexpr int PF_ATT_GROUP = 64;       // tokens per long-context attention launch of the prompt path

struct PfMat { uint8_t *w = nullptr; int type = 0; int64_t n_rows = 0; int nb = 0; };

struct Layer {
    DevMatrix upgate;   // FFN up and gate interleaved in 32-row tiles (when the shard's FFN width is a multiple of 16); else up / gate below
    DevMatrix wqkv, wo, up, gate, down;
    KqSeg     kq_q, kq_k, kq_v, kq_o, kq_up, kq_gate, kq_down;   // K-quant models (Q4_K / Q6_K): the matrices as row ranges in GGUF order
    float    *attn_norm = nullptr, *ffn_norm = nullptr;
    __half   *k_cache = nullptr, *v_cache = nullptr;   // K [n_ctx][dl], V transposed [dl][n_ctx] of the selected sequence
    __half   *k_base = nullptr, *v_base = nullptr;     // the caches of all sequences, seq_stride elements apart (spyb_model_set_sequences)
    // the same weights in the tile layout of the tensor-core prompt kernel (spyb_prefill.cu): Wq|Wk|Wv stacked, up|gate stacked
    PfMat     pf_qkv, pf_wo, pf_ug, pf_down;
    PfMat     pf_k, pf_v, pf_gate;   // K-quant models: one matrix per tensor (types differ per tensor); pf_qkv then holds Wq, pf_ug holds W_up
};

}  // namespace spyb

using namespace spyb;

struct spyb_model {
    spyb_backend   *be = nullptr;
    spyb_model_info info{};
    int             dl = 0, fl = 0;          // local (per-rank) attention width and FFN width
    std::vector<Layer> layers;
    DevMatrix       head;
    KqSeg           kq_head;
    bool            kq = false;              // every matrix is a K-quant: the step plan runs on the K-quant mat-vec kernel
    float          *output_norm = nullptr;
    uint8_t        *embd = nullptr;
    int             embd_type = 0;
    float2         *rope_table = nullptr;
    // activations for up to 8 tokens per pass
    float  *pf_att_scratch = nullptr;   // score rows of a group of prompt tokens at contexts the single-kernel attention serves (the prompt path tiles tokens there too)
    float  *x = nullptr, *att = nullptr, *act = nullptr, *logits = nullptr, *scratch = nullptr, *att_scratch = nullptr;   // att [T][d_model] and act [T][n_ff] are the gathered vectors (inside tp_local)
    __half *q = nullptr;
    int    *d_pos = nullptr;
    int32_t *d_token = nullptr, *d_tokens_in = nullptr, *d_history = nullptr;
    uint8_t *d_tap = nullptr;
    unsigned long long *d_stamps = nullptr;   // profiling aid (SPYB_TIMELINE=1): eight time stamps per kernel of a step
    int    *h_pos_pinned = nullptr; int32_t *h_tok_pinned = nullptr; float *h_logits_pinned = nullptr;
    void   *nccl_comm = nullptr;
    // exchange buffer (exported to the other ranks for the fused all-gather): the gathered attention output [8][d_model] and
    // FFN activation [8][n_ff] as floats, then [2 n_layer sites][tp] flag words, then [sites] CTA counters;
    // tp_peer[r] = rank r's buffer as mapped into this process (tp_peer[tp_rank] = the local one)
    uint8_t *tp_local = nullptr;
    uint8_t *tp_peer[TP_MAX] = {};
    bool     tp_ready = false;
    int      epoch = 0;
    // single-token steps as one persistent kernel (spyb_step.cu) when the shapes allow it
    StepParams  step;
    bool        step_ok = false, step_coop = true;
    int         step_grid = 0, step_ns = 0;
    unsigned long long *d_step_sync = nullptr, *d_step_stamps = nullptr;
    int         step_stamp_count = 0;
    // prompts of SPYB_PREFILL_MIN_TOKENS tokens and more: GEMMs on the tensor cores over chunks of pf_chunk tokens
    bool     pf_ok = false, pf_buffers = false;
    int      pf_chunk = 512;
    int      att_group = TMAX_COLUMNS;   // tokens per attention launch on the long-context path (as many as the score scratch holds)
    float   *pf_x = nullptr, *pf_qkv = nullptr, *pf_att = nullptr, *pf_ug = nullptr, *pf_act = nullptr;
    __half  *pf_q = nullptr;
    uint8_t *pf_yq = nullptr;
    int32_t *pf_tokens = nullptr, *h_pf_tokens = nullptr;
    int     *pf_pos = nullptr, *h_pf_pos = nullptr;      // (first position, positions known to the step) per group of 8 tokens
    // batches of independent sequences in lockstep (spyb_model_set_sequences / spyb_model_decode_batch)
    int      n_seq = 1, cur_seq = 0;
    int64_t  seq_stride = 0;
    float   *logits_batch = nullptr;
    int32_t *batch_tokens = nullptr, *batch_ids = nullptr;
    int64_t  batch_ids_cap = 0;
    cudaGraphExec_t graph_exec = nullptr;
    cudaGraphExec_t graph_eval1 = nullptr;   // single-token spyb_model_eval: staging copies, embedding, layers, head, logits copy
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float   last_ms = 0.f;
    int64_t last_launches = 0, eval1_launches = 0;
    std::vector<void *> owned;
};

namespace {

spyb_status build_step_plan(spyb_model *m);

template <class T>
spyb_status dev_alloc(spyb_model *m, T **p, size_t count) {
    void *raw = nullptr;
    SPYB_CUDA(m->be, cudaMalloc(&raw, count * sizeof(T) + 64));
    SPYB_CUDA(m->be, cudaMemsetAsync(raw, 0, count * sizeof(T) + 64, m->be->stream));
    SPYB_CUDA(m->be, cudaStreamSynchronize(m->be->stream));   // uploads that follow use other streams: order them after the clearing
    m->owned.push_back(raw);
    *p = static_cast<T *>(raw);
    return SPYB_SUCCESS;
}

constexpr int TMAX = TMAX_COLUMNS;   // activation columns the buffers hold

// NCCL form of the exchange (used until the peer buffers are imported): every rank's share [off, off + len) of every
// column is gathered in place into buf [T][stride]; len * tp_size == stride
spyb_status allgather(spyb_model *m, float *buf, int T, int64_t stride, int64_t len, int64_t *launches) {
    if (m->info.tp_size == 1) { return SPYB_SUCCESS; }
    if (m->nccl_comm == nullptr) { m->be->set_error("tensor-parallel model used before spyb_model_init_tp"); return SPYB_FAIL; }
    for (int t = 0; t < T; ++t) {
        float *col = buf + (int64_t)t * stride;
        const int rc = g_nccl.AllGather(col + (int64_t)m->info.tp_rank * len, col, (size_t)len, /*ncclFloat32*/ 7, m->nccl_comm, m->be->stream);
        if (rc != 0) { m->be->set_error("ncclAllGather failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"); return SPYB_FAIL; }
        ++*launches;
    }
    return SPYB_SUCCESS;
}

size_t tp_float_count(const spyb_model *m) { return (size_t)TMAX * ((size_t)m->info.d_model + (size_t)m->info.n_ff); }
size_t tp_buffer_bytes(const spyb_model *m) {
    const size_t sites = 2 * (size_t)m->info.n_layer, n = m->info.tp_size;
    return tp_float_count(m) * 4 + sites * n * 4 + sites * 4 + 256;
}
float *tp_att(const spyb_model *m, uint8_t *base) { return reinterpret_cast<float *>(base); }
float *tp_act(const spyb_model *m, uint8_t *base) { return reinterpret_cast<float *>(base) + (size_t)TMAX * m->info.d_model; }
unsigned *tp_flag(const spyb_model *m, uint8_t *base, size_t site, int rank) {
    return reinterpret_cast<unsigned *>(base + tp_float_count(m) * 4) + site * m->info.tp_size + rank;
}
unsigned *tp_counter(const spyb_model *m, size_t site) {
    const size_t sites = 2 * (size_t)m->info.n_layer, n = m->info.tp_size;
    return reinterpret_cast<unsigned *>(m->tp_local + tp_float_count(m) * 4) + sites * n + site;
}
// producer side of exchange site `site`: this rank's share of the gathered attention output (is_att) or FFN activation
void tp_produce(spyb_model *m, TpLink &l, size_t site, bool is_att) {
    l.n = m->info.tp_size; l.rank = m->info.tp_rank;
    l.stride = is_att ? m->info.d_model : m->info.n_ff;
    l.len = is_att ? m->dl : m->fl; l.off = (int64_t)l.rank * l.len;
    for (int r = 0; r < l.n; ++r) { l.gather[r] = is_att ? tp_att(m, m->tp_peer[r]) : tp_act(m, m->tp_peer[r]); l.flag_out[r] = tp_flag(m, m->tp_peer[r], site, l.rank); }
    l.counter = tp_counter(m, site); l.epoch = m->d_pos + 2;
}
// consumer side: wait until every rank has published its share for this step
void tp_consume(spyb_model *m, TpLink &l, size_t site) {
    l.n = m->info.tp_size; l.rank = m->info.tp_rank;
    l.flag_in = tp_flag(m, m->tp_local, site, 0); l.epoch = m->d_pos + 2;
}

StepMat step_mat_of(const DevMatrix &A) {
    StepMat s;
    s.w = A.w; s.tr = A.tile_rows; s.type = A.type; s.nbp = A.nbp;
    s.n_tiles = (int)(A.n_rows / A.tile_rows);
    s.nrec = A.nbp >> 3;
    s.recb = A.tile_rows * record_row_bytes(A.type);
    s.crecs = std::max(1, std::min(s.nrec, ST_STAGE_BYTES / s.recb));
    s.nch = (s.nrec + s.crecs - 1) / s.crecs;
    return s;
}

// The persistent step kernel serves single-token steps of an unsharded model whose matrices are all in
// fragment-ordered 8- or 16-row tiles (SPYB_STEP=0 keeps the per-matrix kernels).
spyb_status build_step_plan(spyb_model *m) {
    spyb_backend *be = m->be;
    m->step_ok = false;
    if (std::getenv("SPYB_STEP") == nullptr || std::atoi(std::getenv("SPYB_STEP")) == 0) { return SPYB_SUCCESS; }
    if (m->info.tp_size != 1 || m->info.head_dim != 128) { return SPYB_SUCCESS; }
    auto fits = [](const DevMatrix &A) { return A.w != nullptr && A.mma != 0 && (A.tile_rows == 8 || A.tile_rows == 16) && (A.type == 2 || A.type == 8); };
    bool ok = fits(m->head) && (m->info.d_model % 128) == 0 && m->info.d_model <= 4 * 4 * 480;
    for (const Layer &ly : m->layers) { ok = ok && fits(ly.wqkv) && fits(ly.wo) && fits(ly.upgate) && ly.upgate.fused_pair && fits(ly.down); }
    if (!ok) { return SPYB_SUCCESS; }
    std::vector<StepLayer> hl(m->layers.size());
    int nbp_max = m->head.nbp;
    for (size_t L = 0; L < m->layers.size(); ++L) {
        const Layer &ly = m->layers[L];
        hl[L].qkv = step_mat_of(ly.wqkv); hl[L].wo = step_mat_of(ly.wo); hl[L].upgate = step_mat_of(ly.upgate); hl[L].down = step_mat_of(ly.down);
        hl[L].attn_norm = ly.attn_norm; hl[L].ffn_norm = ly.ffn_norm; hl[L].k_cache = ly.k_cache; hl[L].v_cache = ly.v_cache;
        nbp_max = std::max(std::max(nbp_max, ly.wqkv.nbp), std::max(ly.down.nbp, std::max(ly.wo.nbp, ly.upgate.nbp)));
    }
    StepLayer *d_layers = nullptr;
    if (dev_alloc(m, &d_layers, hl.size()) != SPYB_SUCCESS) { return SPYB_FAIL; }
    SPYB_CUDA(be, cudaMemcpy(d_layers, hl.data(), hl.size() * sizeof(StepLayer), cudaMemcpyHostToDevice));
    int8_t *att_q = nullptr; float *att_d = nullptr;
    if (dev_alloc(m, &att_q, (size_t)m->info.d_model) != SPYB_SUCCESS || dev_alloc(m, &att_d, (size_t)m->info.d_model / 32) != SPYB_SUCCESS ||
        dev_alloc(m, &m->d_step_sync, 8) != SPYB_SUCCESS) { return SPYB_FAIL; }
    StepParams &p = m->step;
    p.layers = d_layers; p.n_layer = (int)hl.size(); p.head = step_mat_of(m->head); p.output_norm = m->output_norm;
    p.x = m->x; p.act = m->act; p.logits = m->logits; p.att_q = att_q; p.att_d = att_d; p.q = m->q; p.pos = m->d_pos;
    p.rope = m->rope_table; p.silu_table = be->d_silu_table; p.exp_table = be->d_exp_table;
    p.d = m->info.d_model; p.fl = m->fl; p.n_ctx = m->info.n_ctx; p.n_head = m->info.n_head; p.nbp_max = nbp_max;
    p.eps = m->info.rms_eps; p.att_scale = 1.0f / std::sqrt((float)m->info.head_dim);
    p.sync = m->d_step_sync; p.error_flag = be->d_error_flag; p.wait_limit_ns = be->wait_limit_ns;
    m->step_grid = be->num_sms_total;
    if (const char *v = std::getenv("SPYB_STEP_CTAS")) { const int n = std::atoi(v); if (n > 0 && n <= be->num_sms_total) { m->step_grid = n; } }
    p.att_parts = 4 * p.n_head <= m->step_grid ? 4 : 2 * p.n_head <= m->step_grid ? 2 : 1;
    m->step_ns = step_ring_stages(p, be->smem_optin);
    if (const char *v = std::getenv("SPYB_STEP_STAGES")) { const int n = std::atoi(v); if (n > 15 && n < m->step_ns) { m->step_ns = n; } }
    if (m->step_ns <= 15) { return SPYB_SUCCESS; }   // context too long for the ring that is left: per-matrix kernels
    int resident = 0;
    if (step_resident_ctas(p, m->step_ns, &resident) != cudaSuccess || resident < 1) { cudaGetLastError(); return SPYB_SUCCESS; }
    if (std::getenv("SPYB_TIMELINE") != nullptr) {
        m->step_stamp_count = 16 * p.n_layer + 8;
        if (dev_alloc(m, &m->d_step_stamps, (size_t)2 * m->step_stamp_count) != SPYB_SUCCESS) { return SPYB_FAIL; }
        p.stamps = m->d_step_stamps;
    }
    if (const char *v = std::getenv("SPYB_STEP_COOP")) { m->step_coop = std::atoi(v) != 0; }
    m->step_ok = true;
    return SPYB_SUCCESS;
}

// one single-token step (layers and head) through the persistent kernel
spyb_status run_step(spyb_model *m, bool tap, int64_t *launches) {
    spyb_backend *be = m->be;
    StepParams p = m->step;
    p.tap_xq = tap ? m->d_tap : nullptr;
    p.wait_limit_ns = be->wait_limit_ns;
    SPYB_CUDA(be, cudaMemsetAsync(m->d_step_sync, 0, 32, be->stream));
    SPYB_CUDA(be, launch_step(p, m->step_grid, m->step_ns, m->step_coop, be->stream));
    ++*launches;
    return SPYB_SUCCESS;
}

// the weights of one mat-vec of the step plan: kind 0 = Wq|Wk|Wv, 1 = Wo, 2 = up|gate, 3 = down, 4 = output head
void set_weights(const spyb_model *m, const Layer *ly, int kind, MatvecParams &p) {
    const int d = m->info.d_model;
    if (m->kq) {
        DevMatrix A;   // only the shape is used
        A.type = SPYB_Q4_K; A.k = (kind == 3) ? m->info.n_ff : d; A.nb = (int)(A.k / 32); A.nbp = A.nb;
        switch (kind) {
        case 0: p.kq[0] = ly->kq_q; p.kq[1] = ly->kq_k; p.kq[2] = ly->kq_v; p.kq_n = 3; A.n_rows = 3 * (int64_t)m->dl; break;
        case 1: p.kq[0] = ly->kq_o; p.kq_n = 1; A.n_rows = d; break;
        case 2: p.kq[0] = ly->kq_up; p.kq[1] = ly->kq_gate; p.kq_n = 2; p.pair_mode = 1; A.n_rows = m->fl; break;
        case 3: p.kq[0] = ly->kq_down; p.kq_n = 1; A.n_rows = d; break;
        default: p.kq[0] = m->kq_head; p.kq_n = 1; A.n_rows = m->info.n_vocab; break;
        }
        p.A = A;
        return;
    }
    switch (kind) {
    case 0: p.A = ly->wqkv; break;
    case 1: p.A = ly->wo; break;
    case 2: if (ly->upgate.w) { p.A = ly->upgate; } else { p.A = ly->up; p.B = ly->gate; p.pair_mode = 1; } break;
    case 3: p.A = ly->down; break;
    default: p.A = m->head; break;
    }
}
#ifndef SPYB_NO_MEASUREMENT_AIDS
uint64_t weights_bytes(const MatvecParams &p) {
    if (p.kq_n > 0) {
        uint64_t b = 0;
        for (int i = 0; i < p.kq_n; ++i) { b += (uint64_t)p.kq[i].n_rows * (p.A.k / 256) * (p.kq[i].type == SPYB_Q4_K ? 144 : 210); }
        return b;
    }
    return p.A.bytes() + (p.pair_mode ? p.B.bytes() : 0);
}
#endif

// the five fused kernels of every layer for T tokens whose first position is *d_pos.
// Tensor parallel: Wq|Wk|Wv, attention and FFN up|gate work on this rank's heads / FFN columns; their outputs are
// all-gathered (inside the kernels over peer memory, or by NCCL) and Wo / FFN down run replicated on the complete
// vectors, so no f32 sum is ever split across ranks and every rank holds the single-GPU bits of the residual stream.
// (seq0 >= 0: the T columns are sequences seq0 .. seq0 + T - 1 of a batch in lockstep, each with its own cache)
spyb_status run_layers(spyb_model *m, int T, bool tap, int64_t *launches, int seq0 = -1) {
    spyb_backend *be = m->be;
    const bool pdl = be->config.use_pdl != 0;
    const LaunchCfg cfg = be->launch_cfg(pdl);
    const int d = m->info.d_model, ff = m->info.n_ff, tp = m->info.tp_size, rank = m->info.tp_rank;
    const bool fused = tp > 1 && m->tp_ready;   // exchange through peer memory inside the kernels
    for (size_t L = 0; L < m->layers.size(); ++L) {
        Layer &ly = m->layers[L];
        auto stamps = [&](int k) { return m->d_stamps ? m->d_stamps + 8 * (5 * L + k) : nullptr; };
        {   // 1: norm + quantize -> QKV -> rope + KV append
            MatvecParams p;
            set_weights(m, &ly, 0, p); p.T = T; p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = d; p.norm_w = ly.attn_norm; p.eps = m->info.rms_eps;
            p.epi = EPI_QKV_ROPE; p.pos_base = m->d_pos; p.rope_table = m->rope_table; p.hd = m->info.head_dim; p.dl = m->dl;
            p.q_out = m->q; p.k_cache = ly.k_cache; p.v_cache = ly.v_cache; p.n_ctx = m->info.n_ctx;
            if (seq0 >= 0) { p.seq_stride = m->seq_stride; p.k_cache = ly.k_base + (int64_t)seq0 * m->seq_stride; p.v_cache = ly.v_base + (int64_t)seq0 * m->seq_stride; }
            p.tap_xq = (tap && L == 0) ? m->d_tap : nullptr;
            p.stamps = stamps(0);
            SPYB_CUDA(be, launch_matvec(p, cfg)); ++*launches;
        }
        {   // 2: attention of this rank's heads -> its share of the gathered output
            AttnParams a;
            a.q = m->q; a.k_cache = ly.k_cache; a.v_cache = ly.v_cache; a.out = m->att + (int64_t)rank * m->dl; a.out_stride = d;
            a.pos_base = m->d_pos; a.exp_table = be->d_exp_table;
            a.n_head = m->dl / m->info.head_dim; a.hd = m->info.head_dim; a.dl = m->dl; a.T = T; a.n_ctx = m->info.n_ctx;
            a.scale = 1.0f / std::sqrt((float)m->info.head_dim);
            a.stamps = stamps(1); a.error_flag = be->d_error_flag; a.scratch = m->att_scratch;
            if (seq0 >= 0) { a.seq_stride = m->seq_stride; a.k_cache = ly.k_base + (int64_t)seq0 * m->seq_stride; a.v_cache = ly.v_base + (int64_t)seq0 * m->seq_stride; }
            if (fused) { tp_produce(m, a.tp, 2 * L, true); }
            SPYB_CUDA(be, launch_attention(a, cfg)); ++*launches;
            if (tp > 1 && !fused && allgather(m, m->att, T, d, m->dl, launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
        }
        {   // 3: quantize -> Wo -> + residual (replicated)
            MatvecParams p;
            set_weights(m, &ly, 1, p); p.T = T; p.pro = PRO_QUANT; p.x = m->att; p.x_stride = d;
            p.epi = EPI_RESID; p.resid = m->x; p.out = m->x; p.out_stride = d; p.stamps = stamps(2);
            if (fused) { tp_consume(m, p.tp, 2 * L); }
            SPYB_CUDA(be, launch_matvec(p, cfg)); ++*launches;
        }
        {   // 4: norm + quantize -> up, gate (this rank's FFN columns) -> up * silu(gate) into its share of the gathered activation
            MatvecParams p;
            set_weights(m, &ly, 2, p);
            p.T = T; p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = d; p.norm_w = ly.ffn_norm;
            p.eps = m->info.rms_eps; p.epi = EPI_SILU_MUL; p.out = m->act + (int64_t)rank * m->fl; p.out_stride = ff; p.silu_table = be->d_silu_table;
            p.stamps = stamps(3);
            if (fused) { tp_produce(m, p.tp, 2 * L + 1, false); }
            SPYB_CUDA(be, launch_matvec(p, cfg)); ++*launches;
            if (tp > 1 && !fused && allgather(m, m->act, T, ff, m->fl, launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
        }
        {   // 5: quantize -> Wdown -> + residual (replicated)
            MatvecParams p;
            set_weights(m, &ly, 3, p); p.T = T; p.pro = PRO_QUANT; p.x = m->act; p.x_stride = ff;
            p.epi = EPI_RESID; p.resid = m->x; p.out = m->x; p.out_stride = d; p.stamps = stamps(4);
            if (fused) { tp_consume(m, p.tp, 2 * L + 1); }
            SPYB_CUDA(be, launch_matvec(p, cfg)); ++*launches;
        }
    }
    return SPYB_SUCCESS;
}

// output norm + head on column `col` of x -> logits[n_vocab]
spyb_status run_head(spyb_model *m, int col, int64_t *launches, const float *x_row = nullptr) {
    MatvecParams p;
    set_weights(m, nullptr, 4, p); p.T = 1; p.pro = PRO_NORM_QUANT; p.x = x_row != nullptr ? x_row : m->x + (int64_t)col * m->info.d_model; p.x_stride = m->info.d_model;
    p.norm_w = m->output_norm; p.eps = m->info.rms_eps; p.epi = EPI_STORE; p.out = m->logits; p.out_stride = m->info.n_vocab;
    p.stamps = m->d_stamps ? m->d_stamps + 8 * (5 * m->layers.size()) : nullptr;
    SPYB_CUDA(m->be, launch_matvec(p, m->be->launch_cfg(m->be->config.use_pdl != 0))); ++*launches;
    return SPYB_SUCCESS;
}

// buffers of the tensor-core prompt path, allocated at the first long prompt
spyb_status ensure_prefill_buffers(spyb_model *m) {
    if (m->pf_buffers) { return SPYB_SUCCESS; }
    spyb_backend *be = m->be;
    const size_t C = (size_t)m->pf_chunk, d = m->info.d_model, ff = m->info.n_ff, dl = m->dl;
    const int nb_max = (int)(std::max(d, ff) / 32);
    bool ok = dev_alloc(m, &m->pf_x, C * d) == SPYB_SUCCESS && dev_alloc(m, &m->pf_qkv, C * 3 * dl) == SPYB_SUCCESS && dev_alloc(m, &m->pf_att, C * d) == SPYB_SUCCESS &&
              dev_alloc(m, &m->pf_ug, C * 2 * ff) == SPYB_SUCCESS && dev_alloc(m, &m->pf_act, C * ff) == SPYB_SUCCESS && dev_alloc(m, &m->pf_q, C * dl) == SPYB_SUCCESS &&
              dev_alloc(m, &m->pf_yq, prefill_act_bytes((int)C, nb_max)) == SPYB_SUCCESS && dev_alloc(m, &m->pf_tokens, C) == SPYB_SUCCESS &&
              dev_alloc(m, &m->pf_pos, 2 * (C / TMAX + 1)) == SPYB_SUCCESS;   // (sized for the smallest group)
    if (!ok) { return SPYB_FAIL; }
    // prompts share K rows and V^T rows among tiles of eight tokens at every context length (SPYB_PF_ATT_TILED=0: contexts up to
    // 1024 positions keep one CTA per head and token, as single-token steps do)
    const char *tiled_env = std::getenv("SPYB_PF_ATT_TILED");
    if (m->att_scratch == nullptr && (tiled_env == nullptr || std::atoi(tiled_env) != 0)) {
        const size_t n_pad = ((size_t)m->info.n_ctx + 3) & ~(size_t)3;
        if (dev_alloc(m, &m->pf_att_scratch, (size_t)m->att_group * (dl / m->info.head_dim) * n_pad) != SPYB_SUCCESS) { return SPYB_FAIL; }
    }
    if (cudaMallocHost(reinterpret_cast<void **>(&m->h_pf_tokens), C * 4) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void **>(&m->h_pf_pos), 2 * (C / TMAX + 1) * 4) != cudaSuccess) { be->set_error("pinned host allocation failed"); return SPYB_FAIL; }
    m->pf_buffers = true;
    return SPYB_SUCCESS;
}

// all layers for the T tokens in pf_x (first position d_pos[0], d_pos[1] positions known to the step): per layer
//   norm + quantize -> QKV GEMM -> RoPE / KV append -> attention -> quantize -> Wo GEMM + residual
//   -> norm + quantize -> up|gate GEMM -> up * silu(gate) -> quantize -> down GEMM + residual
// with the arithmetic of the five fused kernels of run_layers, so that a prompt gives the same bits on either path.
// (batch: the T tokens are sequences 0 .. T-1 of a batch in lockstep, each with its own cache, all at position d_pos[0])
spyb_status run_prefill_layers(spyb_model *m, int T, int64_t *launches, bool batch = false) {
    spyb_backend *be = m->be;
    cudaStream_t s = be->stream;
    const LaunchCfg cfg = be->launch_cfg(false);
    const int d = m->info.d_model, ff = m->info.n_ff, dl = m->dl, fl = m->fl, hd = m->info.head_dim;
    const int tp = m->info.tp_size, rank = m->info.tp_rank;
    // the quantized activations are laid out for the type of the matrix they meet (s8 or e4m3 planes, tiles of 16 or 64 tokens):
    // quant() makes them for the first matrix of a group, gemm() makes them again when a later matrix of the group wants another form
    struct { const float *x; int part_len; const float *norm_w; int K; int64_t part_stride; int type; } yq_src = {};
    auto layout_of = [](int type) { return type == SPYB_Q4_K ? 3 : type == SPYB_Q6_K ? 1 : 2; };   // (Q4_0 and Q8_0 share one)
    auto quant = [&](const float *x, int part_len, int K, const float *norm_w, int type, int64_t part_stride) {
        yq_src = {x, part_len, norm_w, K, part_stride, type};
        return launch_prefill_quant(x, part_len, T, K, norm_w, norm_w != nullptr ? m->info.rms_eps : 0.f, m->pf_yq, s, type, part_len, part_stride);
    };
    auto gemm = [&](const PfMat &W, int K, float *out, int64_t out_stride, const float *resid) {
        if (layout_of(W.type) != layout_of(yq_src.type)) {
            cudaError_t e = quant(yq_src.x, yq_src.part_len, yq_src.K, yq_src.norm_w, W.type, yq_src.part_stride);
            if (e != cudaSuccess) { return e; }
            ++*launches;
        }
        PrefillGemm g;
        g.w = W.w; g.type = W.type; g.n_rows = W.n_rows; g.nb = K / 32; g.yq = m->pf_yq; g.T = T; g.out = out; g.out_stride = out_stride; g.resid = resid;
        g.error_flag = be->d_error_flag; g.wait_limit_ns = be->wait_limit_ns;
        return launch_prefill_gemm(g, s);
    };
    // Tensor parallel: every matrix is split by output rows - this rank's heads, FFN rows, and a slice of the rows of W_o and
    // W_down - so each rank produces, for all T tokens, one contiguous part [T][len] of the attention output, the FFN
    // activation and (twice) the residual stream; one NCCL all-gather per vector puts the ranks' parts side by side
    // ([tp][T][len]) and the quantizer in front of the next matrix reads a token's row across the parts. Every dot product
    // is computed whole by one rank: no f32 sum is split across ranks, as on the single-token path.
    auto gather = [&](float *parts, int64_t len) -> spyb_status {
        if (tp == 1) { return SPYB_SUCCESS; }
        if (m->nccl_comm == nullptr) { be->set_error("tensor-parallel model used before spyb_model_init_tp"); return SPYB_FAIL; }
        const size_t count = (size_t)T * len;
        const int rc = g_nccl.AllGather(parts + (size_t)rank * count, parts, count, /*ncclFloat32*/ 7, m->nccl_comm, s);
        if (rc != 0) { be->set_error("ncclAllGather failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"); return SPYB_FAIL; }
        ++*launches;
        return SPYB_SUCCESS;
    };
    const int dp = d / tp;                                  // W_o and W_down: this rank's dp output rows; the residual stream in parts [tp][T][dp]
    float *att_part = m->pf_att + (size_t)rank * T * dl, *act_part = m->pf_act + (size_t)rank * T * fl;   // (tp == 1: the whole buffers)
    float *x_part = m->pf_x + (size_t)rank * T * dp;
    for (Layer &ly : m->layers) {
        SPYB_CUDA(be, quant(m->pf_x, dp, d, ly.attn_norm, ly.pf_qkv.type, (int64_t)T * dp));
        SPYB_CUDA(be, gemm(ly.pf_qkv, d, m->pf_qkv, 3 * (int64_t)dl, nullptr));
        if (m->kq) {   // one matrix per tensor: Wk and Wv fill the other two thirds of the QKV rows
            SPYB_CUDA(be, gemm(ly.pf_k, d, m->pf_qkv + dl, 3 * (int64_t)dl, nullptr));
            SPYB_CUDA(be, gemm(ly.pf_v, d, m->pf_qkv + 2 * dl, 3 * (int64_t)dl, nullptr));
            *launches += 2;
        }
        __half *kc = batch ? ly.k_base : ly.k_cache, *vc = batch ? ly.v_base : ly.v_cache;
        SPYB_CUDA(be, launch_prefill_qkv_post(m->pf_qkv, T, dl, hd, m->d_pos, m->rope_table, m->pf_q, kc, vc, m->info.n_ctx, batch ? m->seq_stride : 0, s));
        *launches += 3;
        AttnParams a;
        a.k_cache = kc; a.v_cache = vc; a.out_stride = dl; a.exp_table = be->d_exp_table; a.seq_stride = batch ? m->seq_stride : 0;
        a.n_head = dl / hd; a.hd = hd; a.dl = dl; a.n_ctx = m->info.n_ctx; a.scale = 1.0f / std::sqrt((float)hd); a.error_flag = be->d_error_flag;
        float *att_rows = m->att_scratch != nullptr ? m->att_scratch : (batch ? nullptr : m->pf_att_scratch);
        if (att_rows == nullptr) {   // short contexts: one CTA per (head, token)
            a.q = m->pf_q; a.out = att_part; a.pos_base = m->d_pos; a.T = T;
            SPYB_CUDA(be, launch_attention(a, cfg)); ++*launches;
        } else {                           // long contexts: the chip-wide kernels on groups of tokens that fit the score scratch
            a.scratch = att_rows; a.force_long = 1;
            for (int t0 = 0; t0 < T; t0 += m->att_group) {
                a.q = m->pf_q + (int64_t)t0 * dl; a.out = att_part + (int64_t)t0 * dl; a.pos_base = batch ? m->d_pos : m->pf_pos + 2 * (t0 / m->att_group); a.T = std::min(m->att_group, T - t0);
                if (batch) { a.k_cache = kc + (int64_t)t0 * m->seq_stride; a.v_cache = vc + (int64_t)t0 * m->seq_stride; }
                SPYB_CUDA(be, launch_attention(a, cfg)); *launches += 3;
            }
        }
        if (gather(m->pf_att, dl) != SPYB_SUCCESS) { return SPYB_FAIL; }
        SPYB_CUDA(be, quant(m->pf_att, dl, d, nullptr, ly.pf_wo.type, (int64_t)T * dl));
        SPYB_CUDA(be, gemm(ly.pf_wo, d, x_part, dp, x_part));
        if (gather(m->pf_x, dp) != SPYB_SUCCESS) { return SPYB_FAIL; }
        SPYB_CUDA(be, quant(m->pf_x, dp, d, ly.ffn_norm, ly.pf_ug.type, (int64_t)T * dp));
        SPYB_CUDA(be, gemm(ly.pf_ug, d, m->pf_ug, 2 * (int64_t)fl, nullptr));
        if (m->kq) { SPYB_CUDA(be, gemm(ly.pf_gate, d, m->pf_ug + fl, 2 * (int64_t)fl, nullptr)); ++*launches; }
        SPYB_CUDA(be, launch_prefill_silu_mul(m->pf_ug, T, fl, be->d_silu_table, act_part, s));
        if (gather(m->pf_act, fl) != SPYB_SUCCESS) { return SPYB_FAIL; }
        SPYB_CUDA(be, quant(m->pf_act, fl, ff, nullptr, ly.pf_down.type, (int64_t)T * fl));
        SPYB_CUDA(be, gemm(ly.pf_down, ff, x_part, dp, x_part));
        if (gather(m->pf_x, dp) != SPYB_SUCCESS) { return SPYB_FAIL; }
        *launches += 7;
    }
    return SPYB_SUCCESS;
}

// output norm + head on the first T columns of x -> out [T][n_vocab]
spyb_status run_head_columns(spyb_model *m, int T, float *out, int64_t *launches) {
    MatvecParams p;
    set_weights(m, nullptr, 4, p); p.T = T; p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = m->info.d_model;
    p.norm_w = m->output_norm; p.eps = m->info.rms_eps; p.epi = EPI_STORE; p.out = out; p.out_stride = m->info.n_vocab;
    SPYB_CUDA(m->be, launch_matvec(p, m->be->launch_cfg(m->be->config.use_pdl != 0))); ++*launches;
    return SPYB_SUCCESS;
}

spyb_status run_decode_step(spyb_model *m, int64_t *launches) {
    if (m->step_ok) {
        if (run_step(m, false, launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
    } else {
        if (run_layers(m, 1, false, launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
        if (run_head(m, 0, launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
    }
    SPYB_CUDA(m->be, launch_argmax_embed(m->logits, m->info.n_vocab, m->d_token, m->d_history, m->d_pos, m->embd, m->embd_type,
                                         m->info.d_model, m->x, m->be->launch_cfg(m->be->config.use_pdl != 0)));
    ++*launches;
    return SPYB_SUCCESS;
}

}  // namespace

extern "C" {

spyb_status spyb_model_load_gguf(spyb_backend *be, const char *path, int32_t n_ctx, spyb_model **out) {
    if (be == nullptr || path == nullptr || out == nullptr) { return SPYB_FAIL; }
    *out = nullptr;
    cudaSetDevice(be->config.device_id);
    GgufFile f; std::string err;
    if (!f.open(path, &err)) { be->set_error("GGUF: %s", err.c_str()); return SPYB_FAIL; }
    if (f.str["general.architecture"] != "llama") { be->set_error("GGUF: architecture '%s' is not supported", f.str["general.architecture"].c_str()); return SPYB_UNSUPPORTED; }
    auto num = [&](const char *k, double dflt) { auto it = f.num.find(k); return it == f.num.end() ? dflt : it->second; };
    spyb_model *m = new spyb_model();
    m->be = be;
    spyb_model_info &I = m->info;
    I.n_layer = (int)num("llama.block_count", 0); I.d_model = (int)num("llama.embedding_length", 0);
    if (const char *cap = std::getenv("SPYB_MAX_LAYERS")) {   // debugging aid: run only the first N blocks of the file
        const int n = std::atoi(cap);
        if (n > 0 && n < I.n_layer) { I.n_layer = n; }
    }
    I.n_head = (int)num("llama.attention.head_count", 0); I.n_ff = (int)num("llama.feed_forward_length", 0);
    I.n_ctx = n_ctx > 0 ? n_ctx : (int)num("llama.context_length", 512);
    I.rms_eps = (float)num("llama.attention.layer_norm_rms_epsilon", 1e-5); I.rope_base = (float)num("llama.rope.freq_base", 10000.0);
    I.tp_size = be->config.tp_size; I.tp_rank = be->config.tp_rank;
    const int kv_heads = (int)num("llama.attention.head_count_kv", I.n_head);
    auto fail = [&](spyb_status st) { spyb_model_free(m); return st; };
    if (I.n_layer <= 0 || I.d_model <= 0 || I.n_head <= 0 || I.n_ff <= 0) { be->set_error("GGUF: missing llama.* hyper-parameters"); return fail(SPYB_FAIL); }
    if (kv_heads != I.n_head) { be->set_error("grouped-query attention (head_count_kv %d != head_count %d) is not supported", kv_heads, I.n_head); return fail(SPYB_UNSUPPORTED); }
    I.head_dim = I.d_model / I.n_head;
    if (I.head_dim != 128) { be->set_error("head_dim %d is not supported (128 only)", I.head_dim); return fail(SPYB_UNSUPPORTED); }
    const int tp = I.tp_size;
    int64_t shard[4];
    if (spyb_tp_layer_shard(I.d_model, I.n_head, I.n_ff, tp, I.tp_rank, shard) != SPYB_SUCCESS) { be->set_error("tp_size %d does not divide heads / FFN blocks", tp); return fail(SPYB_FAIL); }
    m->dl = (int)shard[1]; m->fl = (int)shard[3];
    const int d = I.d_model, dl = m->dl, fl = m->fl, r = I.tp_rank;   // (shard[0] == r * dl, shard[2] == r * fl)

    auto tensor = [&](const std::string &name, const GgufTensor **t, const uint8_t **data) {
        auto it = f.tensors.find(name);
        if (it == f.tensors.end()) { be->set_error("GGUF: tensor %s is missing", name.c_str()); return false; }
        *t = &it->second;
        *data = f.data(it->second, &err);
        if (*data == nullptr) { be->set_error("GGUF: %s: %s", name.c_str(), err.c_str()); return false; }
        return true;
    };
    auto upload_f32 = [&](const std::string &name, int64_t n, float **dst) {
        const GgufTensor *t; const uint8_t *data;
        if (!tensor(name, &t, &data)) { return SPYB_FAIL; }
        if (t->type != SPYB_FP32 || t->ne[0] != n) { be->set_error("GGUF: %s must be f32[%lld]", name.c_str(), (long long)n); return SPYB_FAIL; }
        if (dev_alloc(m, dst, (size_t)n) != SPYB_SUCCESS) { return SPYB_FAIL; }
        SPYB_CUDA(be, cudaMemcpy(*dst, data, (size_t)n * 4, cudaMemcpyHostToDevice));
        return SPYB_SUCCESS;
    };
    // rows [row0, row0 + n_rows) and blocks [blk0, blk0 + nb) of a [k_full, rows_full] matrix -> planes (optionally into `into` at row dst_row)
    auto upload_w = [&](const std::string &name, int64_t k_full, int64_t rows_full, int64_t row0, int64_t n_rows, int64_t blk0, int nb,
                        DevMatrix *dst, DevMatrix *into, int64_t dst_row, int sub_rows = 0, int sub_off = 0) {
        const GgufTensor *t; const uint8_t *data;
        if (!tensor(name, &t, &data)) { return SPYB_FAIL; }
        if (t->ne[0] != k_full || t->ne[1] != rows_full) { be->set_error("GGUF: %s has shape [%lld, %lld]", name.c_str(), (long long)t->ne[0], (long long)t->ne[1]); return SPYB_FAIL; }
        if (t->type != SPYB_Q4_0 && t->type != SPYB_Q8_0) { be->set_error("GGUF: %s: weight type %d has no device kernel", name.c_str(), t->type); return SPYB_UNSUPPORTED; }
        const int64_t rb = GgufFile::row_bytes(t->type, k_full);
        I.weight_bytes += (uint64_t)n_rows * nb * (t->type == SPYB_Q4_0 ? 18 : 34);
        if (into != nullptr) {
            if (into->type != t->type) { be->set_error("GGUF: %s: Wq/Wk/Wv must share one type", name.c_str()); return SPYB_UNSUPPORTED; }
            return upload_matrix(be, t->type, data + row0 * rb, n_rows, rb, blk0, nb, dst, into, dst_row, sub_rows, sub_off);
        }
        return upload_matrix(be, t->type, data + row0 * rb, n_rows, rb, blk0, nb, dst);
    };

    // K-quant matrix: rows [row0, row0 + n_rows) of a [k_full, rows_full] Q4_K / Q6_K tensor, kept in GGUF row order
    auto upload_kq = [&](const std::string &name, int64_t k_full, int64_t rows_full, int64_t row0, int64_t n_rows, KqSeg *dst) {
        const GgufTensor *t; const uint8_t *data;
        if (!tensor(name, &t, &data)) { return SPYB_FAIL; }
        if (t->ne[0] != k_full || t->ne[1] != rows_full) { be->set_error("GGUF: %s has shape [%lld, %lld]", name.c_str(), (long long)t->ne[0], (long long)t->ne[1]); return SPYB_FAIL; }
        if (t->type != SPYB_Q4_K && t->type != SPYB_Q6_K) { be->set_error("GGUF: %s: type %d in a K-quant model (every matrix must be Q4_K or Q6_K)", name.c_str(), t->type); return SPYB_UNSUPPORTED; }
        if (k_full % 256 != 0 || (n_rows & 1)) { be->set_error("GGUF: %s: K-quant rows need K a multiple of 256 and an even row count", name.c_str()); return SPYB_UNSUPPORTED; }
        const int64_t rb_file = GgufFile::row_bytes(t->type, k_full), rb_dev = kq_row_bytes(t->type, k_full);
        uint8_t *dev = nullptr;
        if (dev_alloc(m, &dev, (size_t)n_rows * rb_dev) != SPYB_SUCCESS) { return SPYB_FAIL; }
        if (t->type == SPYB_Q4_K) {
            SPYB_CUDA(be, cudaMemcpy(dev, data + row0 * rb_file, (size_t)n_rows * rb_file, cudaMemcpyHostToDevice));
        } else {   // Q6_K: 210-byte super-blocks -> 16-byte-aligned pieces
            void *stage = nullptr;
            SPYB_CUDA(be, cudaMalloc(&stage, (size_t)n_rows * rb_file + 64));
            // (on the backend's stream, like the kernel that reads it: a plain cudaMemcpy from pageable memory is not
            // ordered with a non-blocking stream)
            cudaError_t err = cudaMemcpyAsync(stage, data + row0 * rb_file, (size_t)n_rows * rb_file, cudaMemcpyHostToDevice, be->stream);
            if (err == cudaSuccess) { err = launch_kq_relayout_q6k(static_cast<const uint8_t *>(stage), n_rows, k_full, dev, be->stream); }
            if (err == cudaSuccess) { err = cudaStreamSynchronize(be->stream); }
            cudaFree(stage);
            if (err != cudaSuccess) { be->set_error("GGUF: %s: upload failed: %s", name.c_str(), cudaGetErrorString(err)); return SPYB_FAIL; }
        }
        dst->w = dev; dst->type = t->type; dst->n_rows = n_rows; dst->row_bytes = rb_dev;
        I.weight_bytes += (uint64_t)n_rows * rb_file;
        return SPYB_SUCCESS;
    };
    // the tile layout of the tensor-core prompt kernel: rows [0, rows_full) of a tensor into rows [dst_row, ...) of a matrix of total_rows rows
    // (rows [row0, row0 + n_rows) of the tensor; n_rows < 0: all of them)
    auto upload_pf = [&](const std::string &name, int64_t k_full, int64_t rows_full, PfMat *into, int64_t dst_row, int64_t total_rows, int64_t row0 = 0, int64_t n_rows = -1) {
        if (n_rows < 0) { n_rows = rows_full; }
        const GgufTensor *t; const uint8_t *data;
        if (!tensor(name, &t, &data)) { return SPYB_FAIL; }
        if (t->ne[0] != k_full || t->ne[1] != rows_full || (t->type != SPYB_Q4_0 && t->type != SPYB_Q8_0 && t->type != SPYB_Q4_K && t->type != SPYB_Q6_K)) { return SPYB_UNSUPPORTED; }
        const int nb = (int)(k_full / 32);
        if (into->w == nullptr) {
            if (dev_alloc(m, &into->w, prefill_weight_bytes(t->type, total_rows, nb)) != SPYB_SUCCESS) { return SPYB_FAIL; }
            into->type = t->type; into->n_rows = total_rows; into->nb = nb;
        } else if (into->type != t->type) { return SPYB_UNSUPPORTED; }
        const int64_t rb = GgufFile::row_bytes(t->type, k_full);
        const int64_t max_rows = std::max<int64_t>(1, (int64_t)(64u << 20) / rb);   // 64 MiB staging pieces
        void *stage = nullptr;
        SPYB_CUDA(be, cudaMalloc(&stage, (size_t)std::min(max_rows, n_rows) * rb + 64));
        for (int64_t r0 = 0; r0 < n_rows; r0 += max_rows) {
            const int64_t nr = std::min(max_rows, n_rows - r0);
            cudaError_t e = cudaMemcpyAsync(stage, data + (row0 + r0) * rb, (size_t)nr * rb, cudaMemcpyHostToDevice, be->stream);
            if (e == cudaSuccess) { e = launch_prefill_retile(t->type, static_cast<const uint8_t *>(stage), rb, nr, nb, into->w, dst_row + r0, be->stream); }
            if (e == cudaSuccess) { e = cudaStreamSynchronize(be->stream); }
            if (e != cudaSuccess) { cudaFree(stage); be->set_error("GGUF: %s: upload failed: %s", name.c_str(), cudaGetErrorString(e)); return SPYB_FAIL; }
        }
        cudaFree(stage);
        return SPYB_SUCCESS;
    };
    {   // a model whose attention query weights are K-quants runs on the K-quant kernel throughout
        auto it = f.tensors.find("blk.0.attn_q.weight");
        m->kq = it != f.tensors.end() && (it->second.type == SPYB_Q4_K || it->second.type == SPYB_Q6_K);
    }

    // embeddings stay in their raw layout (gathered one row at a time); the reference gathers F32 / Q8_0 rows only
    {
        const GgufTensor *t; const uint8_t *data;
        if (!tensor("token_embd.weight", &t, &data)) { return fail(SPYB_FAIL); }
        I.n_vocab = (int)t->ne[1];
        m->embd_type = t->type;
        if (t->type != SPYB_FP32 && t->type != SPYB_FP16 && t->type != SPYB_Q8_0 && t->type != SPYB_Q4_0 && t->type != SPYB_Q4_K && t->type != SPYB_Q6_K) {
            be->set_error("token_embd type %d is not supported", t->type); return fail(SPYB_UNSUPPORTED);
        }
        const size_t bytes = (size_t)GgufFile::row_bytes(t->type, d) * t->ne[1];
        if (dev_alloc(m, &m->embd, bytes) != SPYB_SUCCESS) { return fail(SPYB_FAIL); }
        if (cudaMemcpy(m->embd, data, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { be->set_error("embedding upload failed"); return fail(SPYB_FAIL); }
    }
    spyb_status st = upload_f32("output_norm.weight", d, &m->output_norm);
    if (st != SPYB_SUCCESS) { return fail(st); }
    // tile height per matrix (rows per warp-tile of the mat-vec kernels): 4 = lane-per-accumulator kernel, 8 / 16 / 32 =
    // lane-per-row kernels; the defaults put about one tile on every warp of an SM. SPYB_TILE_<NAME> overrides, and
    // SPYB_NO_ROWS_KERNEL keeps everything on 4-row tiles.
    const bool rows_kernel = std::getenv("SPYB_NO_ROWS_KERNEL") == nullptr;
    auto tile_for = [&](const char *env, int64_t n_rows, int dflt) {
        int t = dflt;
        if (const char *v = std::getenv(env)) { t = std::atoi(v); }
        if (!rows_kernel || (t != 8 && t != 16 && t != 32) || n_rows % t != 0) { t = 4; }
        return t;
    };
    // SPYB_STEP=1: single-token steps as one persistent kernel (needs the fragment-ordered records of the tensor-core
    // kernels); SPYB_MMA=1: tensor-core kernels, one launch per matrix. Default: the byte-dot-product kernels, which
    // measure fastest on the 7B workload (1.63 ms per token against 1.83 / 2.2).
    const bool want_step = std::getenv("SPYB_STEP") != nullptr && std::atoi(std::getenv("SPYB_STEP")) != 0;
    const int  use_mma = (want_step || (std::getenv("SPYB_MMA") != nullptr && std::atoi(std::getenv("SPYB_MMA")) != 0)) ? 1 : 0;
    auto auto_tile = [&](int64_t n_rows) {   // the tallest tile that still gives every SM at least 8 tiles
        const int64_t per_sm = n_rows / std::max(be->num_sms, 1);
        if (use_mma) { return per_sm >= 8 * 16 ? 16 : 8; }
        return per_sm >= 8 * 32 ? 32 : per_sm >= 8 * 16 ? 16 : 8;
    };
    if (m->kq) {
        if ((st = upload_kq("output.weight", d, I.n_vocab, 0, I.n_vocab, &m->kq_head)) != SPYB_SUCCESS) { return fail(st); }
    } else {
        const std::string head_name = f.tensors.count("output.weight") ? "output.weight" : "token_embd.weight";
        auto ith = f.tensors.find(head_name);
        const int head_tile = (I.n_vocab >= 8192 || (use_mma && I.n_vocab % 8 == 0)) ? tile_for("SPYB_TILE_HEAD", I.n_vocab, auto_tile(I.n_vocab)) : 4;
        if (ith != f.tensors.end() && head_tile != 4) {
            DevMatrix dummy;
            if ((st = alloc_matrix(be, ith->second.type, I.n_vocab, d / 32, &m->head, head_tile, use_mma)) != SPYB_SUCCESS) { return fail(st); }
            st = upload_w(head_name, d, I.n_vocab, 0, I.n_vocab, 0, d / 32, &dummy, &m->head, 0);
        } else {
            st = upload_w(head_name, d, I.n_vocab, 0, I.n_vocab, 0, d / 32, &m->head, nullptr, 0);   // replicated on every rank
        }
        if (st != SPYB_SUCCESS) { return fail(st); }
    }
    // prompts run as GEMMs on the tensor cores when the model is unsharded, Q4_0 / Q8_0 throughout and its widths are
    // multiples of the kernel's 128-row tile (SPYB_PREFILL=0 keeps the mat-vec passes; the extra copy of the layer weights is then not made)
    // (a sharded model keeps its rows of every matrix in that layout - its heads, its FFN rows, its slice of the rows of W_o and
    // W_down: the prompt path all-gathers the four vectors of a layer for all tokens of a chunk at once)
    m->pf_ok = (std::getenv("SPYB_PREFILL") == nullptr || std::atoi(std::getenv("SPYB_PREFILL")) != 0) &&
               d <= PF_MAX_K && I.n_ff <= PF_MAX_K && (m->kq ? (tp == 1 && d % 256 == 0 && I.n_ff % 256 == 0) : (dl % 4 == 0 && fl % 4 == 0 && d % (4 * tp) == 0));
    if (const char *v = std::getenv("SPYB_PREFILL_CHUNK")) { const int n = std::atoi(v); if (n >= PF_TOK && n <= 4096) { m->pf_chunk = (n + TMAX - 1) / TMAX * TMAX; } }
    m->layers.resize(I.n_layer);
    for (int L = 0; L < I.n_layer; ++L) {
        Layer &ly = m->layers[L];
        const std::string p = "blk." + std::to_string(L) + ".";
        if ((st = upload_f32(p + "attn_norm.weight", d, &ly.attn_norm)) != SPYB_SUCCESS) { return fail(st); }
        if ((st = upload_f32(p + "ffn_norm.weight", d, &ly.ffn_norm)) != SPYB_SUCCESS) { return fail(st); }
        if (m->kq) {   // K-quants: heads / FFN columns of this rank as row ranges; Wo and W_down whole
            if ((st = upload_kq(p + "attn_q.weight", d, d, (int64_t)r * dl, dl, &ly.kq_q)) != SPYB_SUCCESS || (st = upload_kq(p + "attn_k.weight", d, d, (int64_t)r * dl, dl, &ly.kq_k)) != SPYB_SUCCESS ||
                (st = upload_kq(p + "attn_v.weight", d, d, (int64_t)r * dl, dl, &ly.kq_v)) != SPYB_SUCCESS || (st = upload_kq(p + "attn_output.weight", d, d, 0, d, &ly.kq_o)) != SPYB_SUCCESS ||
                (st = upload_kq(p + "ffn_up.weight", d, I.n_ff, (int64_t)r * fl, fl, &ly.kq_up)) != SPYB_SUCCESS || (st = upload_kq(p + "ffn_gate.weight", d, I.n_ff, (int64_t)r * fl, fl, &ly.kq_gate)) != SPYB_SUCCESS ||
                (st = upload_kq(p + "ffn_down.weight", I.n_ff, d, 0, d, &ly.kq_down)) != SPYB_SUCCESS) { return fail(st); }
            if (dev_alloc(m, &ly.k_cache, (size_t)I.n_ctx * dl) != SPYB_SUCCESS || dev_alloc(m, &ly.v_cache, (size_t)I.n_ctx * dl) != SPYB_SUCCESS) { return fail(SPYB_FAIL); }
            ly.k_base = ly.k_cache; ly.v_base = ly.v_cache;
            if (m->pf_ok) {   // the same tensors in the tile layout of the tensor-core prompt kernel, one matrix per tensor
                spyb_status ps = upload_pf(p + "attn_q.weight", d, d, &ly.pf_qkv, 0, d);
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_k.weight", d, d, &ly.pf_k, 0, d); }
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_v.weight", d, d, &ly.pf_v, 0, d); }
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_output.weight", d, d, &ly.pf_wo, 0, d); }
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_up.weight", d, I.n_ff, &ly.pf_ug, 0, I.n_ff); }
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_gate.weight", d, I.n_ff, &ly.pf_gate, 0, I.n_ff); }
                if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_down.weight", I.n_ff, d, &ly.pf_down, 0, d); }
                if (ps == SPYB_FAIL) { return fail(ps); }
                if (ps != SPYB_SUCCESS) { m->pf_ok = false; }
            }
            continue;
        }
        // heads: rows [r*dl, (r+1)*dl) of Wq, Wk, Wv, stacked into one [3*dl, d] matrix
        auto itq = f.tensors.find(p + "attn_q.weight");
        if (itq == f.tensors.end()) { be->set_error("GGUF: %sattn_q.weight is missing", p.c_str()); return fail(SPYB_FAIL); }
        const int qkv_tile = tile_for("SPYB_TILE_QKV", dl, auto_tile(3 * (int64_t)dl));
        if ((st = alloc_matrix(be, itq->second.type, 3 * (int64_t)dl, d / 32, &ly.wqkv, qkv_tile, use_mma)) != SPYB_SUCCESS) { return fail(st); }
        DevMatrix dummy;
        if ((st = upload_w(p + "attn_q.weight", d, d, (int64_t)r * dl, dl, 0, d / 32, &dummy, &ly.wqkv, 0)) != SPYB_SUCCESS) { return fail(st); }
        if ((st = upload_w(p + "attn_k.weight", d, d, (int64_t)r * dl, dl, 0, d / 32, &dummy, &ly.wqkv, dl)) != SPYB_SUCCESS) { return fail(st); }
        if ((st = upload_w(p + "attn_v.weight", d, d, (int64_t)r * dl, dl, 0, d / 32, &dummy, &ly.wqkv, 2 * (int64_t)dl)) != SPYB_SUCCESS) { return fail(st); }
        // Wo: replicated (all d rows, all d input columns): it consumes the gathered attention output
        auto ito = f.tensors.find(p + "attn_output.weight");
        const int wo_tile = tile_for("SPYB_TILE_WO", d, auto_tile(d));
        if (ito != f.tensors.end() && wo_tile != 4) {
            if ((st = alloc_matrix(be, ito->second.type, d, d / 32, &ly.wo, wo_tile, use_mma)) != SPYB_SUCCESS) { return fail(st); }
            st = upload_w(p + "attn_output.weight", d, d, 0, d, 0, d / 32, &dummy, &ly.wo, 0);
        } else {
            st = upload_w(p + "attn_output.weight", d, d, 0, d, 0, d / 32, &ly.wo, nullptr, 0);
        }
        if (st != SPYB_SUCCESS) { return fail(st); }
        // FFN: rows [r*fl, (r+1)*fl) of up and gate; down is replicated and consumes the gathered activation
        auto itu = f.tensors.find(p + "ffn_up.weight");
        const int ug_tile = tile_for("SPYB_TILE_UPGATE", 2 * (int64_t)fl, auto_tile(2 * (int64_t)fl));
        if (itu != f.tensors.end() && ug_tile != 4) {
            const int half = ug_tile / 2;
            if ((st = alloc_matrix(be, itu->second.type, 2 * (int64_t)fl, d / 32, &ly.upgate, ug_tile, use_mma)) != SPYB_SUCCESS) { return fail(st); }
            ly.upgate.fused_pair = 1;
            if ((st = upload_w(p + "ffn_up.weight", d, I.n_ff, (int64_t)r * fl, fl, 0, d / 32, &dummy, &ly.upgate, 0, half, 0)) != SPYB_SUCCESS) { return fail(st); }
            if ((st = upload_w(p + "ffn_gate.weight", d, I.n_ff, (int64_t)r * fl, fl, 0, d / 32, &dummy, &ly.upgate, 0, half, half)) != SPYB_SUCCESS) { return fail(st); }
        } else {
            if ((st = upload_w(p + "ffn_up.weight", d, I.n_ff, (int64_t)r * fl, fl, 0, d / 32, &ly.up, nullptr, 0)) != SPYB_SUCCESS) { return fail(st); }
            if ((st = upload_w(p + "ffn_gate.weight", d, I.n_ff, (int64_t)r * fl, fl, 0, d / 32, &ly.gate, nullptr, 0)) != SPYB_SUCCESS) { return fail(st); }
            if (ly.up.type != ly.gate.type) { be->set_error("ffn_up and ffn_gate must share one type"); return fail(SPYB_UNSUPPORTED); }
        }
        auto itd = f.tensors.find(p + "ffn_down.weight");
        const int down_tile = tile_for("SPYB_TILE_DOWN", d, auto_tile(d));
        if (itd != f.tensors.end() && down_tile != 4) {
            if ((st = alloc_matrix(be, itd->second.type, d, I.n_ff / 32, &ly.down, down_tile, use_mma)) != SPYB_SUCCESS) { return fail(st); }
            st = upload_w(p + "ffn_down.weight", I.n_ff, d, 0, d, 0, I.n_ff / 32, &dummy, &ly.down, 0);
        } else {
            st = upload_w(p + "ffn_down.weight", I.n_ff, d, 0, d, 0, I.n_ff / 32, &ly.down, nullptr, 0);
        }
        if (st != SPYB_SUCCESS) { return fail(st); }
        if (dev_alloc(m, &ly.k_cache, (size_t)I.n_ctx * dl) != SPYB_SUCCESS || dev_alloc(m, &ly.v_cache, (size_t)I.n_ctx * dl) != SPYB_SUCCESS) { return fail(SPYB_FAIL); }
        ly.k_base = ly.k_cache; ly.v_base = ly.v_cache;
        if (m->pf_ok) {
            const int64_t q0 = (int64_t)r * dl, f0 = (int64_t)r * fl;   // this rank's heads and FFN rows
            spyb_status ps = upload_pf(p + "attn_q.weight", d, d, &ly.pf_qkv, 0, 3 * (int64_t)dl, q0, dl);
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_k.weight", d, d, &ly.pf_qkv, dl, 3 * (int64_t)dl, q0, dl); }
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_v.weight", d, d, &ly.pf_qkv, 2 * (int64_t)dl, 3 * (int64_t)dl, q0, dl); }
            const int64_t dp = d / tp, o0 = (int64_t)r * dp;            // and its slice of the output rows of W_o and W_down
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "attn_output.weight", d, d, &ly.pf_wo, 0, dp, o0, dp); }
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_up.weight", d, I.n_ff, &ly.pf_ug, 0, 2 * (int64_t)fl, f0, fl); }
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_gate.weight", d, I.n_ff, &ly.pf_ug, fl, 2 * (int64_t)fl, f0, fl); }
            if (ps == SPYB_SUCCESS) { ps = upload_pf(p + "ffn_down.weight", I.n_ff, d, &ly.pf_down, 0, dp, o0, dp); }
            if (ps == SPYB_FAIL) { return fail(ps); }
            if (ps != SPYB_SUCCESS) { m->pf_ok = false; }   // a mix of types inside one stacked matrix: prompts stay on the mat-vec passes
        }
    }
    I.weight_bytes += (uint64_t)(2 * I.n_layer + 1) * d * 4;
    I.kv_bytes_per_token = (uint64_t)2 * I.n_layer * dl * 2;
    m->seq_stride = (int64_t)I.n_ctx * dl;

    // RoPE table with the host libm, theta advanced by repeated f32 multiplication exactly as
    // OperatorRopeImpl::execute does (backend/host/operator/non-linear.cpp:282, 300-309)
    {
        const int hd = I.head_dim;
        std::vector<float2> tab((size_t)I.n_ctx * (hd / 2));
        const float theta_scale = std::pow(I.rope_base, -2.0f / (float)hd);
        for (int pos = 0; pos < I.n_ctx; ++pos) {
            float theta = (float)pos;
            for (int i = 0; i < hd / 2; ++i) { tab[(size_t)pos * (hd / 2) + i] = make_float2(std::cos(theta) * 1.0f, std::sin(theta) * 1.0f); theta *= theta_scale; }
        }
        if (dev_alloc(m, &m->rope_table, tab.size()) != SPYB_SUCCESS) { return fail(SPYB_FAIL); }
        if (cudaMemcpy(m->rope_table, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice) != cudaSuccess) { be->set_error("rope table upload failed"); return fail(SPYB_FAIL); }
    }
    {   // the exchange buffer: gathered attention output and FFN activation, flag words, counters (one plain cudaMalloc: it is exported)
        void *raw = nullptr;
        if (cudaMalloc(&raw, tp_buffer_bytes(m)) != cudaSuccess || cudaMemset(raw, 0, tp_buffer_bytes(m)) != cudaSuccess) { be->set_error("exchange buffer allocation failed"); return fail(SPYB_FAIL); }
        m->owned.push_back(raw);
        m->tp_local = static_cast<uint8_t *>(raw);
        m->tp_peer[I.tp_rank] = m->tp_local;
        m->att = tp_att(m, m->tp_local); m->act = tp_act(m, m->tp_local);
    }
    m->att_group = m->pf_ok ? PF_ATT_GROUP : TMAX;
    const size_t att_scratch = attention_scratch_floats(I.n_ctx, dl / I.head_dim, m->att_group);
    bool ok = dev_alloc(m, &m->x, (size_t)TMAX * d) == SPYB_SUCCESS && dev_alloc(m, &m->scratch, (size_t)TMAX * d) == SPYB_SUCCESS &&
              (att_scratch == 0 || dev_alloc(m, &m->att_scratch, att_scratch) == SPYB_SUCCESS) &&
              dev_alloc(m, &m->logits, (size_t)I.n_vocab) == SPYB_SUCCESS && dev_alloc(m, &m->q, (size_t)TMAX * dl) == SPYB_SUCCESS &&
              dev_alloc(m, &m->d_pos, 4) == SPYB_SUCCESS && dev_alloc(m, &m->d_token, 4) == SPYB_SUCCESS &&
              dev_alloc(m, &m->d_tokens_in, TMAX) == SPYB_SUCCESS && dev_alloc(m, &m->d_history, (size_t)I.n_ctx + 8) == SPYB_SUCCESS &&
              dev_alloc(m, &m->d_tap, (size_t)d / 32 * 34) == SPYB_SUCCESS &&
              (std::getenv("SPYB_TIMELINE") == nullptr || dev_alloc(m, &m->d_stamps, (size_t)(5 * I.n_layer + 1) * 8) == SPYB_SUCCESS);
    if (!ok) { return fail(SPYB_FAIL); }
    if (cudaMallocHost(reinterpret_cast<void **>(&m->h_pos_pinned), 64) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void **>(&m->h_tok_pinned), 64) != cudaSuccess ||
        cudaMallocHost(reinterpret_cast<void **>(&m->h_logits_pinned), (size_t)I.n_vocab * 4) != cudaSuccess) {
        be->set_error("pinned host allocation failed"); return fail(SPYB_FAIL);
    }
    if (cudaEventCreate(&m->ev0) != cudaSuccess || cudaEventCreate(&m->ev1) != cudaSuccess) { be->set_error("event creation failed"); return fail(SPYB_FAIL); }
    if (cudaDeviceSynchronize() != cudaSuccess) { be->set_error("device synchronisation after the upload failed"); return fail(SPYB_FAIL); }
    if (build_step_plan(m) != SPYB_SUCCESS) { return fail(SPYB_FAIL); }
    *out = m;
    return SPYB_SUCCESS;
}

void spyb_model_free(spyb_model *m) {
    if (m == nullptr) { return; }
    cudaSetDevice(m->be->config.device_id);
    cudaStreamSynchronize(m->be->stream);
    if (m->graph_exec) { cudaGraphExecDestroy(m->graph_exec); }
    if (m->graph_eval1) { cudaGraphExecDestroy(m->graph_eval1); }
    if (m->nccl_comm && g_nccl.CommDestroy) { g_nccl.CommDestroy(m->nccl_comm); }
    for (void *p : m->owned) { cudaFree(p); }
    if (m->h_pos_pinned) { cudaFreeHost(m->h_pos_pinned); }
    if (m->h_tok_pinned) { cudaFreeHost(m->h_tok_pinned); }
    if (m->h_logits_pinned) { cudaFreeHost(m->h_logits_pinned); }
    if (m->h_pf_tokens) { cudaFreeHost(m->h_pf_tokens); }
    if (m->h_pf_pos) { cudaFreeHost(m->h_pf_pos); }
    if (m->ev0) { cudaEventDestroy(m->ev0); }
    if (m->ev1) { cudaEventDestroy(m->ev1); }
    delete m;
}

spyb_status spyb_model_info_get(const spyb_model *m, spyb_model_info *info) {
    if (m == nullptr || info == nullptr) { return SPYB_FAIL; }
    *info = m->info;
    return SPYB_SUCCESS;
}

spyb_status spyb_nccl_unique_id(void *unique_id_128) {
    if (!g_nccl.load()) { return SPYB_FAIL; }
    return g_nccl.GetUniqueId(unique_id_128) == 0 ? SPYB_SUCCESS : SPYB_FAIL;
}

spyb_status spyb_model_init_tp(spyb_model *m, const void *unique_id_128) {
    if (m == nullptr) { return SPYB_FAIL; }
    if (m->info.tp_size == 1) { return SPYB_SUCCESS; }
    if (!g_nccl.load()) { m->be->set_error("libnccl.so.2 could not be loaded"); return SPYB_FAIL; }
    cudaSetDevice(m->be->config.device_id);
    NcclApi::Uid uid; std::memcpy(uid.b, unique_id_128, 128);
    const int rc = g_nccl.CommInitRank(&m->nccl_comm, m->info.tp_size, uid, m->info.tp_rank);
    if (rc != 0) { m->be->set_error("ncclCommInitRank failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"); return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

spyb_status spyb_model_tp_export(spyb_model *m, void *handle_64) {
    if (m == nullptr || handle_64 == nullptr) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    if (m->info.tp_size < 2 || m->info.tp_size > TP_MAX) { be->set_error("tp_export: tp_size %d", m->info.tp_size); return SPYB_FAIL; }
    cudaSetDevice(be->config.device_id);
    cudaIpcMemHandle_t h;
    SPYB_CUDA(be, cudaIpcGetMemHandle(&h, m->tp_local));
    static_assert(sizeof(h) == 64, "IPC handle size");
    std::memcpy(handle_64, &h, 64);
    return SPYB_SUCCESS;
}

spyb_status spyb_model_tp_import(spyb_model *m, const void *handles) {
    if (m == nullptr || handles == nullptr || m->tp_local == nullptr) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    cudaSetDevice(be->config.device_id);
    for (int r = 0; r < m->info.tp_size; ++r) {
        if (r == m->info.tp_rank) { m->tp_peer[r] = m->tp_local; continue; }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t *>(handles) + 64 * r, 64);
        void *ptr = nullptr;
        SPYB_CUDA(be, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        m->tp_peer[r] = static_cast<uint8_t *>(ptr);
    }
    m->tp_ready = true;
    return SPYB_SUCCESS;
}

spyb_status spyb_model_eval(spyb_model *m, const int32_t *tokens, int32_t n_tokens, int32_t n_past, float *logits_host) {
    if (m == nullptr || tokens == nullptr || n_tokens < 1) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    cudaSetDevice(be->config.device_id);
    if (n_past < 0 || n_past + n_tokens > m->info.n_ctx) { be->set_error("the number of tokens exceeds the context length (%d + %d > %d)", n_past, n_tokens, m->info.n_ctx); return SPYB_FAIL; }
    for (int i = 0; i < n_tokens; ++i) { if (tokens[i] < 0 || tokens[i] >= m->info.n_vocab) { be->set_error("token id %d out of range", tokens[i]); return SPYB_FAIL; } }
    int64_t launches = 0;
    if (n_tokens == 1 && be->config.use_graph != 0 && (m->info.tp_size == 1 || std::getenv("SPYB_TP_NO_GRAPH") == nullptr)) {
        // the host-driven token loop: one captured graph per model (staging words and the logits go through pinned
        // memory whose addresses are fixed, so the graph replays unchanged for every token)
        SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
        m->h_pos_pinned[0] = n_past; m->h_pos_pinned[1] = n_past + 1; m->h_pos_pinned[2] = ++m->epoch;
        m->h_tok_pinned[0] = tokens[0];
        for (int attempt = 0; m->graph_eval1 == nullptr; ++attempt) {
            cudaGraph_t graph = nullptr;
            SPYB_CUDA(be, cudaStreamBeginCapture(be->stream, cudaStreamCaptureModeThreadLocal));
            spyb_status st = SPYB_SUCCESS;
            cudaError_t ce = cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 12, cudaMemcpyHostToDevice, be->stream);
            if (ce == cudaSuccess) { ce = cudaMemcpyAsync(m->d_tokens_in, m->h_tok_pinned, 4, cudaMemcpyHostToDevice, be->stream); }
            if (ce == cudaSuccess) { ce = launch_embed(m->d_tokens_in, 1, m->embd, m->embd_type, m->info.d_model, m->x, be->stream); }
            int64_t n = 1;
            if (ce == cudaSuccess && m->step_ok) { st = run_step(m, true, &n); }
            else {
                if (ce == cudaSuccess) { st = run_layers(m, 1, true, &n); }
                if (ce == cudaSuccess && st == SPYB_SUCCESS) { st = run_head(m, 0, &n); }
            }
            if (ce == cudaSuccess && st == SPYB_SUCCESS) { ce = cudaMemcpyAsync(m->h_logits_pinned, m->logits, (size_t)m->info.n_vocab * 4, cudaMemcpyDeviceToHost, be->stream); }
            const cudaError_t ee = cudaStreamEndCapture(be->stream, &graph);
            cudaError_t ie = cudaSuccess;
            if (ce == cudaSuccess && st == SPYB_SUCCESS && ee == cudaSuccess) {
                ie = cudaGraphInstantiate(&m->graph_eval1, graph, 0);
                if (ie != cudaSuccess) { m->graph_eval1 = nullptr; }
            }
            if (graph) { cudaGraphDestroy(graph); }
            if (m->graph_eval1 != nullptr) { m->eval1_launches = n; break; }
            cudaGetLastError();
            if (attempt == 0 && m->step_ok && m->step_coop) { m->step_coop = false; continue; }   // a cooperative launch the capture refuses: plain launch of the same grid
            if (st == SPYB_SUCCESS) { be->set_error("CUDA graph capture of the single-token step failed: %s", cudaGetErrorString(ce != cudaSuccess ? ce : ee != cudaSuccess ? ee : ie)); }
            return SPYB_FAIL;
        }
        SPYB_CUDA(be, cudaEventRecord(m->ev0, be->stream));
        SPYB_CUDA(be, cudaGraphLaunch(m->graph_eval1, be->stream));
        SPYB_CUDA(be, cudaEventRecord(m->ev1, be->stream));
        SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
        if (be->device_error()) { return SPYB_FAIL; }
        if (logits_host != nullptr) { std::memcpy(logits_host, m->h_logits_pinned, (size_t)m->info.n_vocab * 4); }
        SPYB_CUDA(be, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
        m->last_launches = m->eval1_launches;
        return SPYB_SUCCESS;
    }
    if (m->pf_ok && n_tokens >= SPYB_PREFILL_MIN_TOKENS) {
        // a prompt: chunks of pf_chunk tokens through the tensor-core GEMMs; the score rows of every chunk span all
        // positions known to the step, as in the passes below
        if (ensure_prefill_buffers(m) != SPYB_SUCCESS) { return SPYB_FAIL; }
        SPYB_CUDA(be, cudaEventRecord(m->ev0, be->stream));
        for (int t0 = 0; t0 < n_tokens; t0 += m->pf_chunk) {
            const int T = std::min(m->pf_chunk, n_tokens - t0);
            SPYB_CUDA(be, cudaStreamSynchronize(be->stream));   // pinned staging words are reused per chunk
            m->h_pos_pinned[0] = n_past + t0; m->h_pos_pinned[1] = n_past + n_tokens; m->h_pos_pinned[2] = ++m->epoch;
            std::memcpy(m->h_pf_tokens, tokens + t0, (size_t)T * 4);
            const int groups = (T + m->att_group - 1) / m->att_group;
            for (int gi = 0; gi < groups; ++gi) { m->h_pf_pos[2 * gi] = n_past + t0 + gi * m->att_group; m->h_pf_pos[2 * gi + 1] = n_past + n_tokens; }
            SPYB_CUDA(be, cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 12, cudaMemcpyHostToDevice, be->stream));
            SPYB_CUDA(be, cudaMemcpyAsync(m->pf_pos, m->h_pf_pos, (size_t)groups * 8, cudaMemcpyHostToDevice, be->stream));
            SPYB_CUDA(be, cudaMemcpyAsync(m->pf_tokens, m->h_pf_tokens, (size_t)T * 4, cudaMemcpyHostToDevice, be->stream));
            // sharded: the residual stream of the chunk lives in tp parts [tp][T][d / tp] (rank i produces part i of every token and the
            // parts are all-gathered in place); one part = the plain [T][d]
            const int tp = m->info.tp_size, dmod = m->info.d_model, dp = dmod / tp;
            if (tp == 1) { SPYB_CUDA(be, launch_embed(m->pf_tokens, T, m->embd, m->embd_type, dmod, m->pf_x, be->stream)); ++launches; }
            else {
                SPYB_CUDA(be, launch_embed(m->pf_tokens, T, m->embd, m->embd_type, dmod, m->pf_att, be->stream)); ++launches;
                for (int i = 0; i < tp; ++i) {
                    SPYB_CUDA(be, cudaMemcpy2DAsync(m->pf_x + (size_t)i * T * dp, (size_t)dp * 4, m->pf_att + (size_t)i * dp, (size_t)dmod * 4, (size_t)dp * 4, (size_t)T,
                                                    cudaMemcpyDeviceToDevice, be->stream));
                }
            }
            if (run_prefill_layers(m, T, &launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
            if (t0 + T == n_tokens) {
                const float *last_row = m->pf_x + (int64_t)(T - 1) * dmod;
                if (tp > 1) {   // the last token's row from its parts
                    for (int i = 0; i < tp; ++i) {
                        SPYB_CUDA(be, cudaMemcpyAsync(m->x + (size_t)i * dp, m->pf_x + (size_t)i * T * dp + (size_t)(T - 1) * dp, (size_t)dp * 4, cudaMemcpyDeviceToDevice, be->stream));
                    }
                    last_row = m->x;
                }
                if (run_head(m, 0, &launches, last_row) != SPYB_SUCCESS) { return SPYB_FAIL; }
                if (logits_host != nullptr) {
                    SPYB_CUDA(be, cudaMemcpyAsync(m->h_logits_pinned, m->logits, (size_t)m->info.n_vocab * 4, cudaMemcpyDeviceToHost, be->stream));
                }
            }
        }
        SPYB_CUDA(be, cudaEventRecord(m->ev1, be->stream));
        SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
        if (be->device_error()) { return SPYB_FAIL; }
        if (logits_host != nullptr) { std::memcpy(logits_host, m->h_logits_pinned, (size_t)m->info.n_vocab * 4); }
        SPYB_CUDA(be, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
        m->last_launches = launches;
        return SPYB_SUCCESS;
    }
    SPYB_CUDA(be, cudaEventRecord(m->ev0, be->stream));
    const int tmax = m->kq ? KQ_MAX_COLUMNS : std::min(8, std::min(matvec_max_columns(m->info.d_model / 32), matvec_max_columns(m->info.n_ff / 32)));
    for (int t0 = 0; t0 < n_tokens; t0 += tmax) {
        const int T = std::min(tmax, n_tokens - t0);
        SPYB_CUDA(be, cudaStreamSynchronize(be->stream));   // pinned staging words are reused per pass
        m->h_pos_pinned[0] = n_past + t0;
        m->h_pos_pinned[1] = n_past + n_tokens;   // the step's score rows span every position known to the step
        m->h_pos_pinned[2] = ++m->epoch;          // exchange epoch of this pass (tensor parallel)
        std::memcpy(m->h_tok_pinned, tokens + t0, (size_t)T * 4);
        SPYB_CUDA(be, cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 12, cudaMemcpyHostToDevice, be->stream));
        SPYB_CUDA(be, cudaMemcpyAsync(m->d_tokens_in, m->h_tok_pinned, (size_t)T * 4, cudaMemcpyHostToDevice, be->stream));
        SPYB_CUDA(be, launch_embed(m->d_tokens_in, T, m->embd, m->embd_type, m->info.d_model, m->x, be->stream)); ++launches;
        if (run_layers(m, T, t0 == 0, &launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
        if (t0 + T == n_tokens) {
            if (run_head(m, T - 1, &launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
            if (logits_host != nullptr) {
                SPYB_CUDA(be, cudaMemcpyAsync(m->h_logits_pinned, m->logits, (size_t)m->info.n_vocab * 4, cudaMemcpyDeviceToHost, be->stream));
            }
        }
    }
    SPYB_CUDA(be, cudaEventRecord(m->ev1, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    if (logits_host != nullptr) { std::memcpy(logits_host, m->h_logits_pinned, (size_t)m->info.n_vocab * 4); }
    SPYB_CUDA(be, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    m->last_launches = launches;
    return SPYB_SUCCESS;
}

spyb_status spyb_model_decode(spyb_model *m, int32_t first_token, int32_t n_past, int32_t n_steps, int32_t *ids_host, float *logits_host) {
    if (m == nullptr || n_steps < 1 || ids_host == nullptr) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    cudaSetDevice(be->config.device_id);
    if (n_past < 0 || n_past + n_steps > m->info.n_ctx) { be->set_error("decode would exceed the context length (%d + %d > %d)", n_past, n_steps, m->info.n_ctx); return SPYB_FAIL; }
    if (first_token < 0 || first_token >= m->info.n_vocab) { be->set_error("token id %d out of range", first_token); return SPYB_FAIL; }
    m->h_pos_pinned[0] = n_past; m->h_pos_pinned[1] = 0; *m->h_tok_pinned = first_token;   // [1] = 0: rows end at the token itself
    m->h_pos_pinned[2] = ++m->epoch;   // the argmax kernel advances the device copy once per step
    m->epoch += n_steps - 1;
    SPYB_CUDA(be, cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 12, cudaMemcpyHostToDevice, be->stream));
    SPYB_CUDA(be, cudaMemcpyAsync(m->d_tokens_in, m->h_tok_pinned, 4, cudaMemcpyHostToDevice, be->stream));
    SPYB_CUDA(be, launch_embed(m->d_tokens_in, 1, m->embd, m->embd_type, m->info.d_model, m->x, be->stream));

    const bool use_graph = be->config.use_graph != 0 && (m->info.tp_size == 1 || std::getenv("SPYB_TP_NO_GRAPH") == nullptr);   // the all-reduces of the prompt pass have warmed NCCL up before the capture
    int64_t per_step = 0;
    for (int attempt = 0; use_graph && m->graph_exec == nullptr; ++attempt) {
        // one decode step captured once; positions and the token live in device memory, so the
        // same graph replays for every later step
        cudaGraph_t graph = nullptr;
        SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
        SPYB_CUDA(be, cudaStreamBeginCapture(be->stream, cudaStreamCaptureModeThreadLocal));
        int64_t n = 0;
        const spyb_status st = run_decode_step(m, &n);
        const cudaError_t ce = cudaStreamEndCapture(be->stream, &graph);
        cudaError_t ie = cudaSuccess;
        if (st == SPYB_SUCCESS && ce == cudaSuccess) {
            ie = cudaGraphInstantiate(&m->graph_exec, graph, 0);
            if (ie != cudaSuccess) { m->graph_exec = nullptr; }
        }
        if (graph) { cudaGraphDestroy(graph); }
        if (m->graph_exec != nullptr) { break; }
        cudaGetLastError();
        if (attempt == 0 && m->step_ok && m->step_coop) { m->step_coop = false; continue; }   // a cooperative launch the capture refuses: plain launch of the same grid
        if (st == SPYB_SUCCESS) { be->set_error("CUDA graph capture failed: %s", cudaGetErrorString(ce != cudaSuccess ? ce : ie)); }
        return SPYB_FAIL;
    }
    per_step = m->step_ok ? 2 : (int64_t)m->layers.size() * 5 + 2;
    SPYB_CUDA(be, cudaEventRecord(m->ev0, be->stream));
    for (int s = 0; s < n_steps; ++s) {
        if (use_graph) { SPYB_CUDA(be, cudaGraphLaunch(m->graph_exec, be->stream)); }
        else { int64_t n = 0; if (run_decode_step(m, &n) != SPYB_SUCCESS) { return SPYB_FAIL; } per_step = n; }
        if (logits_host != nullptr) {
            // parity mode: logits of every step come back (argmax_embed does not modify them)
            SPYB_CUDA(be, cudaMemcpyAsync(logits_host + (size_t)s * m->info.n_vocab, m->logits, (size_t)m->info.n_vocab * 4, cudaMemcpyDeviceToHost, be->stream));
            SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
        }
    }
    SPYB_CUDA(be, cudaEventRecord(m->ev1, be->stream));
    SPYB_CUDA(be, cudaMemcpyAsync(ids_host, m->d_history + n_past, (size_t)n_steps * 4, cudaMemcpyDeviceToHost, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    SPYB_CUDA(be, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    m->last_launches = per_step * n_steps;
    return SPYB_SUCCESS;
}

#ifndef SPYB_NO_MEASUREMENT_AIDS
float spyb_model_bench_kernel(spyb_model *m, int32_t kind, int32_t sweeps, uint64_t *bytes_per_launch) {
    if (m == nullptr || kind < 0 || kind > 4 || sweeps < 1) { return -1.f; }
    spyb_backend *be = m->be;
    cudaSetDevice(be->config.device_id);
    const LaunchCfg cfg = be->launch_cfg(false);
    const int d = m->info.d_model;
    m->h_pos_pinned[0] = m->info.n_ctx - 1; m->h_pos_pinned[1] = 0;
    if (cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 8, cudaMemcpyHostToDevice, be->stream) != cudaSuccess) { return -1.f; }
    auto params = [&](const Layer &ly) {
        MatvecParams p; p.T = 1;
        set_weights(m, &ly, kind, p);
        switch (kind) {
        case 0: p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = d; p.norm_w = ly.attn_norm; p.eps = m->info.rms_eps;
                p.epi = EPI_QKV_ROPE; p.pos_base = m->d_pos; p.rope_table = m->rope_table; p.hd = m->info.head_dim; p.dl = m->dl;
                p.q_out = m->q; p.k_cache = ly.k_cache; p.v_cache = ly.v_cache; p.n_ctx = m->info.n_ctx; break;
        case 1: p.pro = PRO_QUANT; p.x = m->att; p.x_stride = d; p.epi = EPI_STORE; p.out = m->scratch; p.out_stride = d; break;
        case 2: p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = d; p.norm_w = ly.ffn_norm;
                p.eps = m->info.rms_eps; p.epi = EPI_SILU_MUL; p.out = m->act + (int64_t)m->info.tp_rank * m->fl; p.out_stride = m->info.n_ff; p.silu_table = be->d_silu_table; break;
        case 3: p.pro = PRO_QUANT; p.x = m->act; p.x_stride = m->info.n_ff; p.epi = EPI_STORE; p.out = m->scratch; p.out_stride = d; break;
        default: p.pro = PRO_NORM_QUANT; p.x = m->x; p.x_stride = d; p.norm_w = m->output_norm; p.eps = m->info.rms_eps;
                p.epi = EPI_STORE; p.out = m->logits; p.out_stride = m->info.n_vocab; break;
        }
        return p;
    };
    const MatvecParams p0 = params(m->layers[0]);
    if (bytes_per_launch) { *bytes_per_launch = weights_bytes(p0); }
    float total_ms = 0.f; int64_t n = 0;
    const bool hot = std::getenv("SPYB_BENCH_L2_HOT") != nullptr;   // every launch on layer 0's matrix: it stays in L2
    if (kind == 4) {
        // a single 70 MB matrix would stay in the 126 MB L2 between launches: every timed launch follows a sweep of the
        // FFN down kernel over the layers' matrices (hundreds of MB), which evicts it
        const int saved_kind = kind;
        for (int s = 0; s < sweeps * 4; ++s) {
            kind = 3;
            for (const Layer &ly : m->layers) { if (launch_matvec(params(ly), cfg) != cudaSuccess) { return -1.f; } }
            kind = saved_kind;
            cudaEventRecord(m->ev0, be->stream);
            if (launch_matvec(p0, cfg) != cudaSuccess) { return -1.f; }
            cudaEventRecord(m->ev1, be->stream);
            cudaStreamSynchronize(be->stream);
            float ms = 0.f; cudaEventElapsedTime(&ms, m->ev0, m->ev1);
            total_ms += ms; ++n;
        }
    } else {
        cudaEventRecord(m->ev0, be->stream);
        for (int s = 0; s < sweeps; ++s) {
            for (const Layer &ly : m->layers) { if (launch_matvec(params(hot ? m->layers[0] : ly), cfg) != cudaSuccess) { return -1.f; } ++n; }
        }
        cudaEventRecord(m->ev1, be->stream);
        if (cudaStreamSynchronize(be->stream) != cudaSuccess) { return -1.f; }
        cudaEventElapsedTime(&total_ms, m->ev0, m->ev1);
    }
    return n ? total_ms / (float)n : -1.f;
}
#endif

spyb_status spyb_tp_layer_shard(int32_t d_model, int32_t n_head, int32_t n_ff, int32_t tp_size, int32_t tp_rank, int64_t out[4]) {
    if (out == nullptr || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size || d_model <= 0 || n_head <= 0 || n_ff <= 0 || d_model % n_head != 0) { return SPYB_FAIL; }
    if (n_head % tp_size != 0 || n_ff % tp_size != 0 || (n_ff / tp_size) % 32 != 0 || (d_model / n_head) % 32 != 0) { return SPYB_FAIL; }
    const int64_t dl = d_model / tp_size, fl = n_ff / tp_size;
    out[0] = (int64_t)tp_rank * dl; out[1] = dl;   // rows of Wq, Wk, Wv = elements of the gathered attention output
    out[2] = (int64_t)tp_rank * fl; out[3] = fl;   // rows of W_up, W_gate = elements of the gathered FFN activation
    return SPYB_SUCCESS;
}

spyb_status spyb_set_wait_limit_ns(spyb_backend *be, uint64_t ns) {
    if (be == nullptr || ns == 0) { return SPYB_FAIL; }
    be->wait_limit_ns = ns;
    return SPYB_SUCCESS;
}

spyb_status spyb_model_selftest_wait_timeout(spyb_model *m, uint64_t limit_ns, int32_t *error_code_out) {
    if (m == nullptr || limit_ns == 0) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    if (!m->step_ok) { be->set_error("selftest: this model does not run on the step kernel"); return SPYB_UNSUPPORTED; }
    cudaSetDevice(be->config.device_id);
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    m->h_pos_pinned[0] = m->info.n_ctx - 1; m->h_pos_pinned[1] = 0;
    SPYB_CUDA(be, cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 8, cudaMemcpyHostToDevice, be->stream));
    StepParams p = m->step;
    p.wait_limit_ns = limit_ns;
    p.barrier_extra = 1;   // every barrier expects one arrival more than there are CTAs: the first one runs out
    SPYB_CUDA(be, cudaMemsetAsync(m->d_step_sync, 0, 32, be->stream));
    SPYB_CUDA(be, launch_step(p, m->step_grid, m->step_ns, m->step_coop, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));   // returns: the kernel ended by itself
    const int code = *reinterpret_cast<volatile int *>(be->h_error_flag);
    if (error_code_out != nullptr) { *error_code_out = code; }
    *reinterpret_cast<volatile int *>(be->h_error_flag) = 0;   // the check leaves the backend usable
    if (code != 2) { be->set_error("selftest: expected the barrier wait to give up with code 2, got %d", code); return SPYB_FAIL; }
    return SPYB_SUCCESS;
}

// ---- batches of independent sequences that share the weights (every step reads them once for all sequences)
static void drop_graphs(spyb_model *m) {
    if (m->graph_exec) { cudaGraphExecDestroy(m->graph_exec); m->graph_exec = nullptr; }
    if (m->graph_eval1) { cudaGraphExecDestroy(m->graph_eval1); m->graph_eval1 = nullptr; }
}

spyb_status spyb_model_set_sequences(spyb_model *m, int32_t n_seq) {
    if (m == nullptr) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    if (n_seq < 1 || n_seq > 64) { be->set_error("set_sequences: 1 to 64 sequences, got %d", n_seq); return SPYB_UNSUPPORTED; }
    if (m->step_ok) { be->set_error("set_sequences: batches need the model on the per-matrix kernels"); return SPYB_UNSUPPORTED; }
    if (m->info.tp_size != 1 && !m->pf_ok) { be->set_error("set_sequences: a sharded model runs batches on the tensor-core kernels, which this model was loaded without"); return SPYB_UNSUPPORTED; }
    cudaSetDevice(be->config.device_id);
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    drop_graphs(m);
    for (Layer &ly : m->layers) {   // fresh caches for all sequences (the previous ones stay allocated until the model is freed)
        if (dev_alloc(m, &ly.k_base, (size_t)n_seq * m->seq_stride) != SPYB_SUCCESS || dev_alloc(m, &ly.v_base, (size_t)n_seq * m->seq_stride) != SPYB_SUCCESS) { return SPYB_FAIL; }
        ly.k_cache = ly.k_base; ly.v_cache = ly.v_base;
    }
    m->n_seq = n_seq; m->cur_seq = 0;
    if (m->logits_batch == nullptr || n_seq > 1) {
        if (dev_alloc(m, &m->logits_batch, (size_t)n_seq * m->info.n_vocab) != SPYB_SUCCESS || dev_alloc(m, &m->batch_tokens, (size_t)n_seq) != SPYB_SUCCESS) { return SPYB_FAIL; }
    }
    return SPYB_SUCCESS;
}

spyb_status spyb_model_select_sequence(spyb_model *m, int32_t seq) {
    if (m == nullptr) { return SPYB_FAIL; }
    if (seq < 0 || seq >= m->n_seq) { m->be->set_error("select_sequence: %d of %d", seq, m->n_seq); return SPYB_FAIL; }
    if (seq == m->cur_seq) { return SPYB_SUCCESS; }
    cudaSetDevice(m->be->config.device_id);
    SPYB_CUDA(m->be, cudaStreamSynchronize(m->be->stream));
    drop_graphs(m);   // the captured steps hold the cache addresses of the sequence they were captured for
    for (Layer &ly : m->layers) { ly.k_cache = ly.k_base + (int64_t)seq * m->seq_stride; ly.v_cache = ly.v_base + (int64_t)seq * m->seq_stride; }
    m->cur_seq = seq;
    return SPYB_SUCCESS;
}

spyb_status spyb_model_decode_batch(spyb_model *m, const int32_t *first_tokens, int32_t n_seq, int32_t n_past, int32_t n_steps, int32_t *ids_host,
                                    float *logits_host) {
    if (m == nullptr || first_tokens == nullptr || ids_host == nullptr || n_steps < 1) { return SPYB_FAIL; }
    spyb_backend *be = m->be;
    cudaSetDevice(be->config.device_id);
    if (n_seq < 1 || n_seq > m->n_seq || m->logits_batch == nullptr) { be->set_error("decode_batch: %d sequences, %d prepared by spyb_model_set_sequences", n_seq, m->n_seq); return SPYB_FAIL; }
    if (n_past < 0 || n_past + n_steps > m->info.n_ctx) { be->set_error("decode would exceed the context length (%d + %d > %d)", n_past, n_steps, m->info.n_ctx); return SPYB_FAIL; }
    for (int c = 0; c < n_seq; ++c) { if (first_tokens[c] < 0 || first_tokens[c] >= m->info.n_vocab) { be->set_error("token id %d out of range", first_tokens[c]); return SPYB_FAIL; } }
    const int64_t need = (int64_t)n_steps * n_seq;
    if (need > m->batch_ids_cap) {
        if (dev_alloc(m, &m->batch_ids, (size_t)need) != SPYB_SUCCESS) { return SPYB_FAIL; }
        m->batch_ids_cap = need;
    }
    const int V = m->info.n_vocab, d = m->info.d_model;
    const int group = m->kq ? KQ_MAX_COLUMNS : std::min(TMAX, std::min(matvec_max_columns(d / 32), matvec_max_columns(m->info.n_ff / 32)));   // columns per pass through the layers
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    m->h_pos_pinned[0] = n_past; m->h_pos_pinned[1] = 0; m->h_pos_pinned[2] = ++m->epoch;
    m->epoch += n_steps - 1;
    SPYB_CUDA(be, cudaMemcpyAsync(m->d_pos, m->h_pos_pinned, 12, cudaMemcpyHostToDevice, be->stream));
    SPYB_CUDA(be, cudaMemcpyAsync(m->batch_tokens, first_tokens, (size_t)n_seq * 4, cudaMemcpyHostToDevice, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));   // (first_tokens may be pageable: it is consumed here)
    int64_t launches = 0;
    SPYB_CUDA(be, cudaEventRecord(m->ev0, be->stream));
    // enough sequences to fill the tensor-core tiles; a sharded model always takes that path (its all-gathers of whole vectors)
    const int  tp   = m->info.tp_size, dp = d / tp;
    const bool gemm = m->pf_ok && n_seq <= m->pf_chunk && (n_seq >= SPYB_PREFILL_MIN_TOKENS || tp > 1);
    if (tp > 1 && !gemm) { be->set_error("decode_batch: a sharded model takes at most %d sequences", m->pf_chunk); return SPYB_UNSUPPORTED; }
    if (gemm && ensure_prefill_buffers(m) != SPYB_SUCCESS) { return SPYB_FAIL; }
    for (int step = 0; step < n_steps; ++step) {
        if (gemm) {   // the sequences of a step are the "tokens" of one GEMM pass; the head runs on groups of columns
            if (tp == 1) { SPYB_CUDA(be, launch_embed(m->batch_tokens, n_seq, m->embd, m->embd_type, d, m->pf_x, be->stream)); ++launches; }
            else {        // the residual stream in tp parts [tp][n_seq][d / tp], as for a prompt
                SPYB_CUDA(be, launch_embed(m->batch_tokens, n_seq, m->embd, m->embd_type, d, m->pf_att, be->stream)); ++launches;
                for (int i = 0; i < tp; ++i) {
                    SPYB_CUDA(be, cudaMemcpy2DAsync(m->pf_x + (size_t)i * n_seq * dp, (size_t)dp * 4, m->pf_att + (size_t)i * dp, (size_t)d * 4, (size_t)dp * 4, (size_t)n_seq,
                                                    cudaMemcpyDeviceToDevice, be->stream));
                }
            }
            if (run_prefill_layers(m, n_seq, &launches, true) != SPYB_SUCCESS) { return SPYB_FAIL; }
            for (int g0 = 0; g0 < n_seq; g0 += group) {
                const int T = std::min(group, n_seq - g0);
                for (int i = 0; i < tp; ++i) {   // whole rows of the group's columns from their parts
                    SPYB_CUDA(be, cudaMemcpy2DAsync(m->x + (size_t)i * dp, (size_t)d * 4, m->pf_x + (size_t)i * n_seq * dp + (size_t)g0 * dp, (size_t)dp * 4, (size_t)dp * 4, (size_t)T,
                                                    cudaMemcpyDeviceToDevice, be->stream));
                }
                if (run_head_columns(m, T, m->logits_batch + (int64_t)g0 * V, &launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
            }
        }
        for (int g0 = 0; !gemm && g0 < n_seq; g0 += group) {
            const int T = std::min(group, n_seq - g0);
            SPYB_CUDA(be, launch_embed(m->batch_tokens + g0, T, m->embd, m->embd_type, d, m->x, be->stream)); ++launches;
            if (run_layers(m, T, false, &launches, g0) != SPYB_SUCCESS) { return SPYB_FAIL; }
            if (run_head_columns(m, T, m->logits_batch + (int64_t)g0 * V, &launches) != SPYB_SUCCESS) { return SPYB_FAIL; }
        }
        SPYB_CUDA(be, launch_argmax_embed_batch(m->logits_batch, V, n_seq, m->batch_tokens, m->batch_ids + (int64_t)step * n_seq, nullptr, 0, d, nullptr, 0, m->d_pos, be->stream));
        launches += 2;
        if (logits_host != nullptr) {
            SPYB_CUDA(be, cudaMemcpyAsync(logits_host + (int64_t)step * n_seq * V, m->logits_batch, (size_t)n_seq * V * 4, cudaMemcpyDeviceToHost, be->stream));
        }
    }
    SPYB_CUDA(be, cudaEventRecord(m->ev1, be->stream));
    SPYB_CUDA(be, cudaMemcpyAsync(ids_host, m->batch_ids, (size_t)need * 4, cudaMemcpyDeviceToHost, be->stream));
    SPYB_CUDA(be, cudaStreamSynchronize(be->stream));
    if (be->device_error()) { return SPYB_FAIL; }
    SPYB_CUDA(be, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    m->last_launches = launches;
    return SPYB_SUCCESS;
}

float   spyb_model_last_ms(const spyb_model *m) { return m ? m->last_ms : 0.f; }
int64_t spyb_model_last_launches(const spyb_model *m) { return m ? m->last_launches : 0; }

spyb_status spyb_model_read_activation(spyb_model *m, int32_t which, void *host, uint64_t bytes) {
    if (m == nullptr || host == nullptr) { return SPYB_FAIL; }
    const void *src = nullptr; uint64_t avail = 0;
    switch (which) {
    case 0: src = m->q;      avail = (uint64_t)8 * m->dl * 2; break;
    case 1: src = m->att;    avail = (uint64_t)8 * m->info.d_model * 4; break;
    case 2: src = m->x;      avail = (uint64_t)8 * m->info.d_model * 4; break;
    case 3: src = m->act;    avail = (uint64_t)8 * m->info.n_ff * 4; break;
    case 4: src = m->logits; avail = (uint64_t)m->info.n_vocab * 4; break;
    default: m->be->set_error("read_activation: unknown buffer %d", which); return SPYB_FAIL;
    }
    if (bytes > avail) { m->be->set_error("read_activation: %llu bytes requested, %llu available", (unsigned long long)bytes, (unsigned long long)avail); return SPYB_FAIL; }
    SPYB_CUDA(m->be, cudaStreamSynchronize(m->be->stream));
    SPYB_CUDA(m->be, cudaMemcpy(host, src, bytes, cudaMemcpyDeviceToHost));
    return SPYB_SUCCESS;
}

#ifndef SPYB_NO_MEASUREMENT_AIDS
int32_t spyb_model_read_timeline(spyb_model *m, uint64_t *stamps_host, int32_t max_kernels) {
    if (m == nullptr || m->d_stamps == nullptr || stamps_host == nullptr) { return 0; }
    const int n = std::min<int>(max_kernels, 5 * (int)m->layers.size() + 1);
    if (cudaMemcpy(stamps_host, m->d_stamps, (size_t)n * 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost) != cudaSuccess) { return 0; }
    return n;
}

int32_t spyb_model_read_step_timeline(spyb_model *m, uint64_t *stamps_host, int32_t max_points) {
    if (m == nullptr || m->d_step_stamps == nullptr || stamps_host == nullptr) { return 0; }
    const int n = std::min<int>(max_points, m->step_stamp_count);
    if (cudaMemcpy(stamps_host, m->d_step_stamps, (size_t)n * 2 * sizeof(uint64_t), cudaMemcpyDeviceToHost) != cudaSuccess) { return 0; }
    return n;
}
#endif

spyb_status spyb_model_tap_xq(spyb_model *m, void *blocks_host) {
    if (m == nullptr || blocks_host == nullptr) { return SPYB_FAIL; }
    SPYB_CUDA(m->be, cudaMemcpy(blocks_host, m->d_tap, (size_t)m->info.d_model / 32 * 34, cudaMemcpyDeviceToHost));
    return SPYB_SUCCESS;
}

}  // extern "C"
