// Launching a kernel handle from raw device pointers: the C counterpart of what the reference's runner does
// with a PTX entry point -- `cuModuleLoadData` on the text compile.py printed, then `cuLaunchKernel` with one
// pointer per parameter in meta.json's `arg_order`, buffers as device pointers and scalars by value
// (tools/run_local.py:64-72, :80-102; parameter list: emmyptx/kernel.py:166-183). Here the text is a kernel handle
// (JSON: entry, variant, parameters, arg_order), "loading" it is parsing it, and the launch is a call of the entry
// point that implements the variant. A runner that holds `cuMemAlloc` pointers needs nothing else from this
// repository: no Python, no torch.
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace emmy {
namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true / false / null) ---------------------------
struct JVal {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    double num = 0.0;
    bool flag = false;
    std::string str;
    std::vector<JVal> items;
    std::map<std::string, JVal> fields;

    const JVal* get(const char* key) const {
        auto it = fields.find(key);
        return it == fields.end() ? nullptr : &it->second;
    }
    bool is_num() const { return kind == Num; }
    int64_t as_int(int64_t fallback = 0) const { return kind == Num ? (int64_t)num : (kind == Bool ? (flag ? 1 : 0) : fallback); }
    bool truthy() const { return kind == Bool ? flag : (kind == Num ? num != 0.0 : (kind == Str ? !str.empty() : kind != Null)); }
};

struct JReader {
    const char* p;
    const char* end;
    bool ok = true;

    void skip() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { skip(); if (p < end && *p == c) { ++p; return true; } return false; }

    JVal value(int depth = 0) {
        JVal v;
        skip();
        if (p >= end || depth > 32) { ok = false; return v; }
        const char c = *p;
        if (c == '{') {
            ++p; v.kind = JVal::Obj;
            if (eat('}')) return v;
            do {
                JVal k = value(depth + 1);
                if (k.kind != JVal::Str || !eat(':')) { ok = false; return v; }
                v.fields[k.str] = value(depth + 1);
            } while (ok && eat(','));
            if (!eat('}')) ok = false;
        } else if (c == '[') {
            ++p; v.kind = JVal::Arr;
            if (eat(']')) return v;
            do { v.items.push_back(value(depth + 1)); } while (ok && eat(','));
            if (!eat(']')) ok = false;
        } else if (c == '"') {
            ++p; v.kind = JVal::Str;
            while (p < end && *p != '"') {
                if (*p == '\\' && p + 1 < end) { ++p; v.str += (*p == 'n' ? '\n' : (*p == 't' ? '\t' : *p)); }
                else v.str += *p;
                ++p;
            }
            if (p >= end) ok = false; else ++p;
        } else if (!strncmp(p, "true", 4)) { p += 4; v.kind = JVal::Bool; v.flag = true; }
        else if (!strncmp(p, "false", 5)) { p += 5; v.kind = JVal::Bool; v.flag = false; }
        else if (!strncmp(p, "null", 4)) { p += 4; }
        else if (!strncmp(p, "NaN", 3)) { p += 3; v.kind = JVal::Num; v.num = strtod("nan", nullptr); }
        else if (!strncmp(p, "Infinity", 8)) { p += 8; v.kind = JVal::Num; v.num = strtod("inf", nullptr); }
        else if (!strncmp(p, "-Infinity", 9)) { p += 9; v.kind = JVal::Num; v.num = -strtod("inf", nullptr); }
        else {
            char* stop = nullptr;
            v.num = strtod(p, &stop);
            if (stop == p) { ok = false; return v; }
            v.kind = JVal::Num;
            p = stop;
        }
        return v;
    }
};

bool parse_handle(const char* text, JVal* out) {
    if (text == nullptr) return false;
    JReader r{text, text + strlen(text)};
    *out = r.value();
    return r.ok && out->kind == JVal::Obj && out->get("variant") != nullptr && out->get("params") != nullptr &&
           out->get("arg_order") != nullptr && out->get("inputs") != nullptr && out->get("outputs") != nullptr;
}

int index_of(const JVal& list, const std::string& name) {
    for (size_t i = 0; i < list.items.size(); ++i)
        if (list.items[i].kind == JVal::Str && list.items[i].str == name) return (int)i;
    return -1;
}

}  // namespace
}  // namespace emmy

namespace emmy {
namespace {

int code_of(const char* const* names, int count, const std::string& name) {
    for (int i = 0; i < count; ++i)
        if (name == names[i]) return i;
    return -1;
}

const char* const kPointwiseOps[] = {"exp_sin_tanh", "exp", "sin", "cos", "tanh", "gelu_tanh", "sigmoid", "silu", "relu"};
const char* const kProgramOps[] = {"add", "subtract", "multiply", "divide", "maximum", "minimum", "relu", "square", "copy", "negative",
                                   "abs", "reciprocal", "sqrt", "rsqrt", "exp", "log", "sigmoid", "tanh", "erf", "sin", "cos", "pow",
                                   "equal", "not_equal", "greater", "less", "greater_equal", "less_equal", "where", "bitwise_and",
                                   "bitwise_or", "bitwise_not", "floor_divide", "mod", "bitwise_xor", "left_shift", "right_shift"};
struct RowOp { const char* name; int code; };
const RowOp kRowOps[] = {{"sum", EMMYB200_ROW_SUM}, {"mean", EMMYB200_ROW_MEAN}, {"amax", EMMYB200_ROW_AMAX}, {"amin", EMMYB200_ROW_AMIN},
                         {"prod", EMMYB200_ROW_PROD}, {"var", EMMYB200_ROW_VAR}, {"std", EMMYB200_ROW_STD}, {"norm2", EMMYB200_ROW_NORM2},
                         {"logsumexp", EMMYB200_ROW_LOGSUMEXP}, {"argmax", EMMYB200_ROW_ARGMAX}, {"dot", EMMYB200_ROW_DOT},
                         {"cosine", EMMYB200_ROW_COSINE}, {"softmax", EMMYB200_ROW_SOFTMAX}, {"log_softmax", EMMYB200_ROW_LOG_SOFTMAX},
                         {"layer_norm", EMMYB200_ROW_LAYER_NORM}, {"rms_norm", EMMYB200_ROW_RMS_NORM}, {"normalize", EMMYB200_ROW_NORMALIZE}};

int dtype_code(const std::string& d) {
    if (d == "f32") return EMMYB200_F32;
    if (d == "f16") return EMMYB200_F16;
    if (d == "bf16") return EMMYB200_BF16;
    if (d == "i32" || d == "int") return EMMYB200_I32;
    if (d == "i64") return EMMYB200_I64;
    if (d == "bool" || d == "u8") return EMMYB200_U8;
    return -1;
}

int row_op_code(const std::string& name) {
    for (const RowOp& r : kRowOps)
        if (name == r.name) return r.code;
    return -1;
}

int epilogue_code(const JVal* e) {
    if (e == nullptr || e->kind == JVal::Null) return EMMYB200_EPI_NONE;
    if (e->kind != JVal::Str) return -1;
    if (e->str == "none" || e->str.empty()) return EMMYB200_EPI_NONE;
    if (e->str == "gelu_tanh") return EMMYB200_EPI_GELU_TANH;
    if (e->str == "relu") return EMMYB200_EPI_RELU;
    return -1;
}

// The handle's arguments as the caller passed them: params[i] points at the value of arg_order[i].
struct Args {
    const JVal& handle;
    void* const* params;
    int n;

    // device pointer of buffer `name`, or null with the error text set
    void* buffer(const std::string& name) const {
        const int i = index_of(*handle.get("arg_order"), name);
        if (i < 0 || i >= n || params[i] == nullptr) return nullptr;
        return *reinterpret_cast<void* const*>(params[i]);
    }
    void* input(size_t k) const {
        const JVal& in = *handle.get("inputs");
        return k < in.items.size() ? buffer(in.items[k].str) : nullptr;
    }
    void* output() const {
        const JVal& out = *handle.get("outputs");
        return out.items.empty() ? nullptr : buffer(out.items[0].str);
    }
};

int64_t geti(const JVal& p, const char* key, int64_t fallback = 0) {
    const JVal* v = p.get(key);
    return v == nullptr ? fallback : v->as_int(fallback);
}
bool getb(const JVal& p, const char* key) {
    const JVal* v = p.get(key);
    return v != nullptr && v->truthy();
}
double getd(const JVal& p, const char* key, double fallback = 0.0) {
    const JVal* v = p.get(key);
    return v != nullptr && v->is_num() ? v->num : fallback;
}
std::string gets(const JVal& p, const char* key) {
    const JVal* v = p.get(key);
    return v != nullptr && v->kind == JVal::Str ? v->str : std::string();
}

bool is_row_map(int op) { return op >= EMMYB200_ROW_SOFTMAX; }

// Fills the C program struct from the handle's "program" object; scalar arguments of the launch (passed by value, as
// the reference passes `.param .f32 / .s32`, emmyptx/kernel.py:171-178) land in the constant slots the matcher reserved.
int fill_program(const JVal& prog, const Args& args, emmyb200_pw_program* out) {
    memset(out, 0, sizeof(*out));
    const JVal* in_dtypes = prog.get("in_dtypes");
    const JVal* steps = prog.get("steps");
    const JVal* consts = prog.get("consts");
    if (in_dtypes == nullptr || steps == nullptr || consts == nullptr) return fail(EMMYB200_ERR_ARG, "launch: the handle's program is incomplete");
    if (in_dtypes->items.size() > EMMYB200_PW_MAX_INPUTS || steps->items.size() > EMMYB200_PW_MAX_STEPS || consts->items.size() > EMMYB200_PW_MAX_CONSTS)
        return fail(EMMYB200_ERR_ARG, "launch: the handle's program exceeds the kernel's limits");
    out->n_inputs = (int32_t)in_dtypes->items.size();
    out->n_steps = (int32_t)steps->items.size();
    out->out_slot = (int32_t)geti(prog, "out_slot");
    out->out_dtype = dtype_code(gets(prog, "out_dtype"));
    const JVal* in_div = prog.get("in_div");
    const JVal* in_mod = prog.get("in_mod");
    for (size_t i = 0; i < in_dtypes->items.size(); ++i) {
        out->in_dtype[i] = dtype_code(in_dtypes->items[i].str);
        if (out->in_dtype[i] < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown input dtype in the handle");
        if (in_div != nullptr && i < in_div->items.size()) out->in_div[i] = in_div->items[i].as_int();
        if (in_mod != nullptr && i < in_mod->items.size()) out->in_mod[i] = in_mod->items[i].as_int();
    }
    if (out->out_dtype < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown output dtype in the handle");
    for (size_t i = 0; i < consts->items.size(); ++i) out->consts[i] = (float)consts->items[i].num;
    const bool trunc = gets(prog, "int_div") == "trunc";
    for (size_t i = 0; i < steps->items.size(); ++i) {
        const JVal& st = steps->items[i];
        if (st.items.size() != 5 || st.items[0].kind != JVal::Str) return fail(EMMYB200_ERR_ARG, "launch: malformed program step");
        std::string op = st.items[0].str;
        if (op == "exp_fast") op = "exp";
        if (op == "remainder") op = "mod";
        const int code = code_of(kProgramOps, (int)(sizeof(kProgramOps) / sizeof(kProgramOps[0])), op);
        if (code < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown program op '%s'", op.c_str());
        out->steps[i].op = (uint8_t)code;
        out->steps[i].dst = (uint8_t)st.items[1].as_int();
        out->steps[i].a = (uint8_t)st.items[2].as_int();
        out->steps[i].b = (uint8_t)st.items[3].as_int();
        out->steps[i].c = (uint8_t)st.items[4].as_int();
        out->steps[i].reserved[0] = trunc ? 1 : 0;
    }
    if (const JVal* sc = prog.get("scalar_consts")) {
        for (const JVal& e : sc->items) {                       // [argument name, constant index, "f32" | "s32"]
            if (e.items.size() != 3) return fail(EMMYB200_ERR_ARG, "launch: malformed scalar binding");
            const int i = index_of(*args.handle.get("arg_order"), e.items[0].str);
            const int64_t slot = e.items[1].as_int();
            if (i < 0 || i >= args.n || args.params[i] == nullptr || slot < 0 || slot >= EMMYB200_PW_MAX_CONSTS)
                return fail(EMMYB200_ERR_ARG, "launch: scalar argument '%s' is missing", e.items[0].str.c_str());
            out->consts[slot] = e.items[2].str == "f32" ? *reinterpret_cast<const float*>(args.params[i])
                                                         : (float)*reinterpret_cast<const int32_t*>(args.params[i]);
        }
    }
    return EMMYB200_OK;
}

}  // namespace
}  // namespace emmy

// Workspace a launch of the handle needs (bytes of 256-byte-aligned device memory; 0 for most variants).
extern "C" int64_t emmyb200_launch_workspace_bytes(const char* handle_json) {
    using namespace emmy;
    JVal h;
    if (!parse_handle(handle_json, &h)) return -1;
    const JVal& p = *h.get("params");
    const std::string v = gets(h, "variant");
    if (v == "gemm_f32")
        return emmyb200_gemm_f32_workspace_bytes(getb(p, "b_trans") ? EMMYB200_GEMM_B_NK : 0, geti(p, "batch", 1), geti(p, "m"), geti(p, "n"),
                                                 geti(p, "k"), getb(p, "b_shared") ? 1 : 0);
    if (v == "rowwise_f32") return emmyb200_rowwise_workspace_bytes(row_op_code(gets(p, "op")), geti(p, "rows"), geti(p, "cols"));
    if (v == "colwise_f32") return emmyb200_colwise_workspace_bytes(row_op_code(gets(p, "op")), geti(p, "outer", 1), geti(p, "rows"), geti(p, "cols"));
    return 0;
}

extern "C" int emmyb200_launch(const char* handle_json, void* const* params, int n_params, void* workspace, int64_t workspace_bytes,
                               void* cuda_stream) {
    using namespace emmy;
    JVal h;
    if (!parse_handle(handle_json, &h)) return fail(EMMYB200_ERR_ARG, "launch: the text is not a kernel handle");
    const JVal& order = *h.get("arg_order");
    if (params == nullptr || n_params != (int)order.items.size())
        return fail(EMMYB200_ERR_ARG, "launch: %d parameters given, the handle's arg_order has %d", n_params, (int)order.items.size());
    const JVal& p = *h.get("params");
    const std::string v = gets(h, "variant");
    const Args a{h, params, n_params};
    for (const char* list : {"inputs", "outputs"})
        for (const JVal& name : h.get(list)->items)
            if (a.buffer(name.str) == nullptr) return fail(EMMYB200_ERR_ARG, "launch: buffer '%s' is null or not in arg_order", name.str.c_str());
    void* out = a.output();
    if (v == "pointwise_f32") {
        const int op = code_of(kPointwiseOps, (int)(sizeof(kPointwiseOps) / sizeof(kPointwiseOps[0])), gets(p, "op"));
        if (op < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown pointwise op");
        return emmyb200_pointwise_f32(op, (const float*)a.input(0), (float*)out, geti(p, "n"), cuda_stream);
    }
    if (v == "pointwise_program") {
        const JVal* prog = p.get("program");
        if (prog == nullptr) return fail(EMMYB200_ERR_ARG, "launch: the handle has no program");
        emmyb200_pw_program c;
        int rc = fill_program(*prog, a, &c);
        if (rc != EMMYB200_OK) return rc;
        const void* ins[EMMYB200_PW_MAX_INPUTS] = {nullptr, nullptr, nullptr, nullptr};
        for (int i = 0; i < c.n_inputs; ++i) ins[i] = a.input(i);
        return emmyb200_pointwise_program(&c, ins, out, geti(p, "n"), cuda_stream);
    }
    if (v == "pointwise_indexed") {
        const JVal* prog = p.get("program");
        const JVal* im = p.get("index_map");
        if (prog == nullptr || im == nullptr) return fail(EMMYB200_ERR_ARG, "launch: the handle has no program or no index map");
        emmyb200_pw_program c;
        int rc = fill_program(*prog, a, &c);
        if (rc != EMMYB200_OK) return rc;
        const JVal* ext = im->get("extents");
        const JVal* srcs = im->get("inputs");
        const JVal* dst = im->get("out");
        if (ext == nullptr || srcs == nullptr || dst == nullptr || ext->items.empty() || ext->items.size() > EMMYB200_PW_MAX_AXES ||
            (int)srcs->items.size() != c.n_inputs || dst->get("coef") == nullptr || dst->get("coef")->items.size() != ext->items.size())
            return fail(EMMYB200_ERR_ARG, "launch: malformed index map");
        emmyb200_pw_index_map m;
        memset(&m, 0, sizeof m);
        m.n_axes = (int)ext->items.size();
        for (int ax = 0; ax < m.n_axes; ++ax) {
            m.extent[ax] = ext->items[ax].as_int();
            m.out_coef[ax] = dst->get("coef")->items[ax].as_int();
        }
        m.out_offset = geti(*dst, "offset");
        const void* ins[EMMYB200_PW_MAX_INPUTS] = {nullptr, nullptr, nullptr, nullptr};
        int next_buffer = 0;                                  // the handle's inputs are the buffer-backed sources, in program order
        for (int k = 0; k < c.n_inputs; ++k) {
            const JVal& src = srcs->items[k];
            if (src.get("axis") != nullptr) {
                m.in_kind[k] = 1;
                m.in_axis[k] = (int)geti(src, "axis");
                continue;
            }
            const JVal* coef = src.get("coef");
            if (coef == nullptr || (int)coef->items.size() != m.n_axes) return fail(EMMYB200_ERR_ARG, "launch: malformed index map");
            m.in_offset[k] = geti(src, "offset");
            for (int ax = 0; ax < m.n_axes; ++ax) m.in_coef[k][ax] = coef->items[ax].as_int();
            if (const JVal* rot = src.get("rot"))
                for (int ax = 0; ax < m.n_axes && ax < (int)rot->items.size(); ++ax) m.in_rot[k][ax] = rot->items[ax].as_int();
            if (src.get("index_mod") != nullptr) {                  // an index source
                m.in_kind[k] = 3;
                m.in_index_mod[k] = geti(src, "index_mod");
                m.in_index_abs[k] = getb(src, "index_abs") ? 1 : 0;
            } else if (src.get("index_of") != nullptr) {            // addressed through an index source
                m.in_kind[k] = 2;
                m.in_index_of[k] = (int)geti(src, "index_of");
                m.in_index_mult[k] = geti(src, "index_mult");
            } else if (src.get("clamp") != nullptr) {               // a guarded read, clamped into the buffer
                m.in_kind[k] = 4;
                m.in_index_mod[k] = geti(src, "clamp");
            }
            if (next_buffer >= (int)h.get("inputs")->items.size()) return fail(EMMYB200_ERR_ARG, "launch: the index map names more buffers than the handle has inputs");
            ins[k] = a.input(next_buffer++);
        }
        return emmyb200_pointwise_indexed(&c, &m, ins, out, cuda_stream);
    }
    if (v == "contract_indexed") {
        const JVal* cm = p.get("map");
        const JVal* ext = cm ? cm->get("extents") : nullptr;
        const JVal* loops = cm ? cm->get("loops") : nullptr;
        const JVal* dst = cm ? cm->get("out") : nullptr;
        if (ext == nullptr || loops == nullptr || dst == nullptr || cm->get("a") == nullptr || cm->get("b") == nullptr || ext->items.empty() ||
            ext->items.size() > EMMYB200_PW_MAX_AXES || loops->items.empty() || loops->items.size() > EMMYB200_CT_MAX_LOOPS)
            return fail(EMMYB200_ERR_ARG, "launch: malformed contraction map");
        emmyb200_contraction_map m;
        memset(&m, 0, sizeof m);
        m.n_axes = (int)ext->items.size();
        m.n_loops = (int)loops->items.size();
        for (int ax = 0; ax < m.n_axes; ++ax) m.extent[ax] = ext->items[ax].as_int();
        for (int l = 0; l < m.n_loops; ++l) m.loop_extent[l] = loops->items[l].as_int();
        auto side = [&](const JVal& src, int64_t* offset, int64_t* coef, int64_t* loop_coef, int* dtype) -> bool {
            const JVal* c = src.get("coef");
            const JVal* lc = src.get("loop_coef");
            if (c == nullptr || (int)c->items.size() != m.n_axes || (loop_coef != nullptr && (lc == nullptr || (int)lc->items.size() != m.n_loops))) return false;
            *offset = geti(src, "offset");
            for (int ax = 0; ax < m.n_axes; ++ax) coef[ax] = c->items[ax].as_int();
            for (int l = 0; loop_coef != nullptr && l < m.n_loops; ++l) loop_coef[l] = lc->items[l].as_int();
            *dtype = dtype_code(gets(src, "dtype"));
            return true;
        };
        if (!side(*cm->get("a"), &m.a_offset, m.a_coef, m.a_loop_coef, &m.a_dtype) || !side(*cm->get("b"), &m.b_offset, m.b_coef, m.b_loop_coef, &m.b_dtype) ||
            !side(*dst, &m.out_offset, m.out_coef, nullptr, &m.out_dtype))
            return fail(EMMYB200_ERR_ARG, "launch: malformed contraction map");
        return emmyb200_contract_indexed(&m, a.input(0), a.input(1), out, cuda_stream);
    }
    if (v == "index_gather_i32")
        return emmyb200_index_gather_i32((const int32_t*)a.input(0), (int32_t*)out, geti(p, "n"), geti(p, "mul"), geti(p, "add"), (int32_t)geti(p, "div"),
                                         (int32_t)geti(p, "shift"), getb(p, "trunc") ? EMMYB200_GATHER_TRUNC : 0, cuda_stream);
    if (v == "gemm" || v == "gemm_batched" || v == "gemm_f32") {
        const int epi = epilogue_code(p.get("epilogue"));
        if (epi < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown epilogue in the handle");
        const int64_t m = geti(p, "m"), n = geti(p, "n"), k = geti(p, "k"), batch = geti(p, "batch", 1);
        const bool nk = getb(p, "b_trans");
        const int flags = (nk ? EMMYB200_GEMM_B_NK : 0) | (getb(p, "out_f32") ? EMMYB200_GEMM_OUT_F32 : 0);
        const int64_t ldb = nk ? k : n;
        if (v == "gemm") return emmyb200_gemm(dtype_code(gets(p, "dtype")), epi, flags, a.input(0), a.input(1), out, m, n, k, k, ldb, n, cuda_stream);
        const void* bias = getb(p, "bias") ? a.input(2) : nullptr;
        const int64_t stride_b = getb(p, "b_shared") ? 0 : (nk ? n : k) * ldb;
        if (v == "gemm_batched")
            return emmyb200_gemm_batched(dtype_code(gets(p, "dtype")), epi, flags, a.input(0), a.input(1), bias, out, batch, m, n, k, k, ldb, n, m * k,
                                         stride_b, m * n, cuda_stream);
        return emmyb200_gemm_f32(epi, flags, (const float*)a.input(0), (const float*)a.input(1), (const float*)bias, (float*)out, batch, m, n, k, k, ldb,
                                 n, batch > 1 ? m * k : 0, batch > 1 ? stride_b : 0, batch > 1 ? m * n : 0, workspace, workspace_bytes, cuda_stream);
    }
    if (v == "attention_fwd")
        return emmyb200_attention_fwd(dtype_code(gets(p, "dtype")), getb(p, "causal") ? EMMYB200_ATT_CAUSAL : 0, a.input(0), a.input(1), a.input(2), out,
                                      geti(p, "units"), geti(p, "seq_q"), geti(p, "seq_k"), geti(p, "d"), (float)getd(p, "scale"), cuda_stream);
    if (v == "rowwise_f32" || v == "colwise_f32") {
        const int op = row_op_code(gets(p, "op"));
        if (op < 0) return fail(EMMYB200_ERR_ARG, "launch: unknown row op in the handle");
        if (v == "rowwise_f32")
            return emmyb200_rowwise_f32(op, (const float*)a.input(0), getb(p, "weight") ? (const float*)a.input(1) : nullptr,
                                        getb(p, "bias") ? (const float*)a.input(2) : nullptr, out, geti(p, "rows"), geti(p, "cols"), (float)getd(p, "eps"),
                                        workspace, workspace_bytes, cuda_stream);
        return emmyb200_colwise_f32(op, (const float*)a.input(0), out, geti(p, "outer", 1), geti(p, "rows"), geti(p, "cols"), (float)getd(p, "eps"),
                                    workspace, workspace_bytes, cuda_stream);
    }
    return fail(EMMYB200_ERR_UNSUPPORTED, "launch: unknown kernel variant '%s'", v.c_str());
}
