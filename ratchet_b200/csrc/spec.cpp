// Host-side rules of the Matmul node (see spec.hpp).  No CUDA here.
#include "spec.hpp"

#include <algorithm>
#include <sstream>

namespace rt {

static thread_local std::string g_last_error;

void set_last_error(const std::string &m) { g_last_error = m; }
const std::string &last_error() { return g_last_error; }

rt_status fail(rt_status code, const std::string &m) {
    g_last_error = m;
    return code;
}
rt_status fail(const Status &s) { return fail(s.code, s.msg); }

Dims to_dims(const rt_shape &s) {
    Dims d;
    for (int i = 0; i < s.rank && i < RT_MAX_RANK; i++) d.push_back(s.dims[i]);
    return d;
}

bool from_dims(const Dims &d, rt_shape *s) {
    if (d.size() > RT_MAX_RANK) return false;
    s->rank = (int32_t)d.size();
    for (int i = 0; i < RT_MAX_RANK; i++) s->dims[i] = i < (int)d.size() ? d[i] : 0;
    return true;
}

std::string dims_str(const Dims &d) {
    std::ostringstream o;
    o << "[";
    for (size_t i = 0; i < d.size(); i++) o << (i ? "," : "") << d[i];
    o << "]";
    return o.str();
}

bool is_vector(const Dims &d) {
    int non_unit = 0;
    for (auto v : d) non_unit += (v != 1);
    return non_unit <= 1;
}

bool multi_broadcast(const Dims &a, const Dims &b, Dims *out) {
    size_t rank = std::max(a.size(), b.size());
    Dims r(rank, 1);
    for (size_t i = 0; i < rank; i++) {
        int64_t cur = 1;
        for (const Dims *s : {&a, &b}) {
            int64_t dim = i < s->size() ? (*s)[s->size() - i - 1] : 1;
            if (dim != 1) {
                if (cur != 1 && dim != cur) return false;
                cur = dim;
            }
        }
        r[rank - i - 1] = cur;
    }
    *out = r;
    return true;
}

bool dtype_valid(int dt) { return dt >= RT_F32 && dt <= RT_Q4_K; }
bool is_quantized(rt_dtype dt) { return dt == RT_Q8_0H || dt == RT_Q8_0F || dt == RT_Q4_K; }

const char *dtype_name(rt_dtype dt) {
    switch (dt) {
    case RT_F32: return "F32";
    case RT_F16: return "F16";
    case RT_BF16: return "BF16";
    case RT_I32: return "I32";
    case RT_U32: return "U32";
    case RT_Q8_0H: return "Q8_0H";
    case RT_Q8_0F: return "Q8_0F";
    case RT_Q4_K: return "Q4_K";
    }
    return "?";
}

size_t dtype_size(rt_dtype dt) {
    switch (dt) {
    case RT_F32: case RT_I32: case RT_U32: return 4;
    case RT_F16: case RT_BF16: return 2;
    default: return 0;
    }
}

rt_dtype activation_dt(rt_dtype dt) {
    switch (dt) {
    case RT_Q8_0H: return RT_F16;
    case RT_Q8_0F: return RT_F32;
    case RT_Q4_K: return RT_F16;
    default: return dt;
    }
}

// Matmul::compute_c_shape (ops/matmul.rs:284-361).  `full` (optional) receives the shape
// with the implicit unit dims kept, which is what the stacking logic works on.
static Status c_shape_impl(const Dims &a_in, const Dims &b_in, bool tl, bool tr, bool to, Dims *out,
                           Dims *a_full, Dims *b_full, Dims *c_full) {
    Dims a = a_in, b = b_in;
    if (a.empty() || b.empty())
        return Status::Err(RT_ERR_SHAPE, "Matmul: rank-0 operand");
    for (auto v : a) if (v < 0) return Status::Err(RT_ERR_SHAPE, "negative extent");
    for (auto v : b) if (v < 0) return Status::Err(RT_ERR_SHAPE, "negative extent");
    bool implicit_m = a.size() < 2, implicit_n = b.size() < 2;
    if (implicit_m) a.insert(a.begin() + (tl ? 1 : 0), 1);
    if (implicit_n) b.insert(b.begin() + (tr ? 0 : 1), 1);
    while (a.size() < b.size()) a.insert(a.begin(), 1);
    while (b.size() < a.size()) b.insert(b.begin(), 1);
    size_t rank = a.size();
    Dims ap(a.begin(), a.end() - 2), bp(b.begin(), b.end() - 2), prefix;
    if (!multi_broadcast(ap, bp, &prefix))
        return Status::Err(RT_ERR_SHAPE, "Matmul broadcasting: a: " + dims_str(a) + " b: " + dims_str(b));
    int64_t m = a[rank - 2], ka = a[rank - 1], kb = b[rank - 2], n = b[rank - 1];
    if (tl) std::swap(m, ka);
    if (tr) std::swap(kb, n);
    if (ka != kb) {
        std::ostringstream o;
        o << "Matmul broadcasting: ka != kb: " << ka << " != " << kb;
        return Status::Err(RT_ERR_SHAPE, o.str());
    }
    Dims c = prefix, cf = prefix;
    if (to) {
        cf.push_back(n); cf.push_back(m);
        if (!implicit_n) c.push_back(n);
        if (!implicit_m) c.push_back(m);
    } else {
        cf.push_back(m); cf.push_back(n);
        if (!implicit_m) c.push_back(m);
        if (!implicit_n) c.push_back(n);
    }
    if (out) *out = c;
    if (a_full) *a_full = a;
    if (b_full) *b_full = b;
    if (c_full) *c_full = cf;
    return Status::Ok();
}

Status compute_c_shape(const Dims &a, const Dims &b, bool tl, bool tr, bool to, Dims *out) {
    return c_shape_impl(a, b, tl, tr, to, out, nullptr, nullptr, nullptr);
}

// OpGuards::check_dtypes (ops/matmul.rs:454-477).  The first four pairs are the reference's;
// the others are this library's extensions (bf16 activations, Q4_K weights, f32-scaled Q8_0
// with f16 activations).
static bool pair_allowed(rt_dtype l, rt_dtype r) {
    static const rt_dtype pairs[][2] = {
        {RT_F32, RT_F32}, {RT_F16, RT_F16}, {RT_Q8_0F, RT_F32}, {RT_Q8_0H, RT_F16},
        {RT_BF16, RT_BF16}, {RT_Q8_0H, RT_BF16}, {RT_Q4_K, RT_F16}, {RT_Q4_K, RT_BF16},
        {RT_Q8_0F, RT_F16},
    };
    for (auto &p : pairs)
        if (p[0] == l && p[1] == r) return true;
    return false;
}

Status resolve_spec(const rt_matmul_desc &d, Spec *s) {
    if (!dtype_valid(d.lhs_dt) || !dtype_valid(d.rhs_dt) || (d.has_bias && !dtype_valid(d.bias_dt)))
        return Status::Err(RT_ERR_ARG, "invalid dtype enum");
    if (d.lhs_shape.rank < 0 || d.lhs_shape.rank > RT_MAX_RANK || d.rhs_shape.rank < 0 ||
        d.rhs_shape.rank > RT_MAX_RANK)
        return Status::Err(RT_ERR_ARG, "rank out of range");
    if (d.epilogue != RT_EPILOGUE_NONE && d.epilogue != RT_EPILOGUE_GELU_TANH && d.epilogue != RT_EPILOGUE_SILU_MUL)
        return Status::Err(RT_ERR_ARG, "invalid epilogue");
    Dims a = to_dims(d.lhs_shape), b = to_dims(d.rhs_shape);
    bool tl = d.trans_lhs != 0, tr = d.trans_rhs != 0, to = d.trans_out != 0;

    // Matmul::new (ops/matmul.rs:258-282)
    Dims bias_dims;
    if (d.has_bias) {
        if (d.bias_shape.rank < 0 || d.bias_shape.rank > RT_MAX_RANK)
            return Status::Err(RT_ERR_ARG, "rank out of range");
        bias_dims = to_dims(d.bias_shape);
        if (!is_vector(bias_dims))
            return Status::Err(RT_ERR_INVARIANT, "Bias must be a vector: " + dims_str(bias_dims));
    }
    if (is_quantized(d.lhs_dt) && tl)
        return Status::Err(RT_ERR_INVARIANT, "Transposed quantized inputs are not supported");

    // OpGuards::check_shapes
    Dims c, af, bf, cf;
    Status st = c_shape_impl(a, b, tl, tr, to, &c, &af, &bf, &cf);
    if (!st.ok()) return st;

    // OpGuards::check_dtypes
    if (!pair_allowed(d.lhs_dt, d.rhs_dt))
        return Status::Err(RT_ERR_DTYPE, std::string("Failed to validate DTypes: ") + dtype_name(d.lhs_dt) +
                                             ", " + dtype_name(d.rhs_dt));
    if (d.has_bias && d.bias_dt != d.rhs_dt && !(d.bias_dt == RT_F16 && d.rhs_dt == RT_BF16))
        return Status::Err(RT_ERR_DTYPE, std::string("Failed to validate DTypes: bias ") +
                                             dtype_name(d.bias_dt) + ", rhs " + dtype_name(d.rhs_dt));

    // GEMMSpec::new (ops/matmul.rs:53-134): drain the leading dims into stack counts
    size_t rank = cf.size();
    size_t stack_dims = rank - 2;
    s->desc = d;
    s->out_shape = c;
    s->out_dt = d.rhs_dt;
    s->lhs_stack = s->rhs_stack = s->out_stack = 1;
    for (size_t i = 0; i < stack_dims; i++) {
        s->lhs_stack *= af[i];
        s->rhs_stack *= bf[i];
        s->out_stack *= cf[i];
    }
    s->stacks = s->out_stack;
    if (s->lhs_stack != 1 && s->rhs_stack != 1 &&
        !(s->lhs_stack == s->rhs_stack && s->rhs_stack == s->out_stack))
        return Status::Err(RT_ERR_INVARIANT,
                           "Matmul stacking: batch dims must be equal or broadcast from 1: " + dims_str(af) +
                               " x " + dims_str(bf));
    // a side whose stack is 1 broadcasts; a side with stack == out_stack indexes directly
    if ((s->lhs_stack != 1 && s->lhs_stack != s->out_stack) || (s->rhs_stack != 1 && s->rhs_stack != s->out_stack))
        return Status::Err(RT_ERR_INVARIANT,
                           "Matmul stacking: batch dims must be equal or broadcast from 1: " + dims_str(af) +
                               " x " + dims_str(bf));
    s->lhs2 = Dims(af.end() - 2, af.end());
    s->rhs2 = Dims(bf.end() - 2, bf.end());
    s->out2 = Dims(cf.end() - 2, cf.end());
    s->trans_lhs = tl; s->trans_rhs = tr; s->trans_out = to;
    s->M = tl ? s->lhs2[1] : s->lhs2[0];
    s->K = tl ? s->lhs2[0] : s->lhs2[1];
    s->N = tr ? s->rhs2[0] : s->rhs2[1];
    s->is_gemv = is_vector(s->rhs2) && !tl; // GEMMSpec::is_gemv (ops/matmul.rs:221-223)
    s->has_bias = d.has_bias != 0;
    s->epilogue = d.epilogue;
    s->bias_len = 0;
    if (s->has_bias) {
        s->bias_len = numel(bias_dims);
        // gemm.rs:468-476: bias indexes the lhs row when trans_out, else the rhs column.
        // gemv.rs:476-490 always indexes the lhs row, so a GEMV accepts a length-M bias too.
        int64_t want = to ? s->M : s->N;
        bool gemv_rowwise = (s->N == 1 && !tl && s->bias_len == s->M);
        if (s->bias_len != want && !gemv_rowwise) {
            std::ostringstream o;
            o << "Bias length " << s->bias_len << " does not match the output dimension " << want;
            return Status::Err(RT_ERR_SHAPE, o.str());
        }
    }
    // gate/up pairs (phi3/mlp.rs:31-39): the Linear node's last output extent is the 2*ff rows of W, which the
    // epilogue folds into ff
    if (d.epilogue == RT_EPILOGUE_SILU_MUL) {
        if (!(to && tr && !tl))
            return Status::Err(RT_ERR_INVARIANT, "RT_EPILOGUE_SILU_MUL takes the Linear form (trans_rhs, trans_out) only");
        if (s->M % 2 != 0)
            return Status::Err(RT_ERR_SHAPE, "RT_EPILOGUE_SILU_MUL needs an even number of weight rows (gate | up)");
        s->out_shape.back() = s->M / 2;
    }
    // block formats run along K inside a row (dtype/blocks.rs:61-74; gemm.rs:111,123)
    if ((d.lhs_dt == RT_Q8_0H || d.lhs_dt == RT_Q8_0F) && s->K % 32 != 0)
        return Status::Err(RT_ERR_SHAPE, "Q8_0 needs the inner dimension to be a multiple of 32");
    if (d.lhs_dt == RT_Q4_K && s->K % 256 != 0)
        return Status::Err(RT_ERR_SHAPE, "Q4_K needs the inner dimension to be a multiple of 256");
    // MatmulMeta holds i32 extents (ops/matmul.rs:375-387)
    for (int64_t v : {s->M, s->N, s->K, s->stacks})
        if (v >= (int64_t(1) << 31)) return Status::Err(RT_ERR_SHAPE, "extent exceeds i32");
    return Status::Ok();
}

void fill_public_spec(const Spec &s, rt_gemm_spec *o) {
    from_dims(s.out_shape, &o->out_shape);
    o->out_dt = s.out_dt;
    o->lhs_stack = s.lhs_stack;
    o->rhs_stack = s.rhs_stack;
    o->out_stack = s.out_stack;
    o->stacks = s.stacks;
    o->dim_lhs_outer = s.M;
    o->dim_rhs_outer = s.N;
    o->dim_inner = s.K;
    o->is_gemv = s.is_gemv ? 1 : 0;
}

} // namespace rt
