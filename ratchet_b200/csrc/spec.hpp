// Host-side rules of the Matmul node: shapes, dtypes, stacking, routing.
// Restates crates/ratchet-core/src/ops/matmul.rs:53-361,442-478 and
// crates/ratchet-core/src/shape.rs:71-136 of the reference; no CUDA in this file.
#pragma once
#include <string>
#include <vector>

#include "ratchet_b200.h"

namespace rt {

struct Status {
    rt_status code = RT_OK;
    std::string msg;
    bool ok() const { return code == RT_OK; }
    static Status Ok() { return {}; }
    static Status Err(rt_status c, std::string m) { return {c, std::move(m)}; }
};

void set_last_error(const std::string &m);
const std::string &last_error();
rt_status fail(rt_status code, const std::string &m);
rt_status fail(const Status &s);

using Dims = std::vector<int64_t>;

inline int64_t numel(const Dims &d) {
    int64_t n = 1;
    for (auto v : d) n *= v;
    return n;
}
Dims to_dims(const rt_shape &s);
bool from_dims(const Dims &d, rt_shape *s);
std::string dims_str(const Dims &d);

// Shape::is_vector (shape.rs:71-75): at most one extent differs from 1.
bool is_vector(const Dims &d);
// Shape::multi_broadcast (shape.rs:118-136) for two shapes; false when incompatible.
bool multi_broadcast(const Dims &a, const Dims &b, Dims *out);

bool dtype_valid(int dt);
bool is_quantized(rt_dtype dt);
const char *dtype_name(rt_dtype dt);
size_t dtype_size(rt_dtype dt);
// activation dtype of a weight dtype (dtype/mod.rs:77-83); Q4_K pairs with f16.
rt_dtype activation_dt(rt_dtype dt);

// The resolved node: everything a kernel launch needs to know about the problem.
struct Spec {
    rt_matmul_desc desc{};
    Dims out_shape;           // compute_c_shape
    rt_dtype out_dt = RT_F32; // rhs dtype
    Dims lhs2, rhs2, out2;    // the trailing two dims after draining the stack dims
    int64_t lhs_stack = 1, rhs_stack = 1, out_stack = 1, stacks = 1;
    int64_t M = 0, N = 0, K = 0; // rows of op(lhs), cols of op(rhs), inner
    bool is_gemv = false;
    bool trans_lhs = false, trans_rhs = false, trans_out = false, has_bias = false;
    int64_t bias_len = 0;
    int epilogue = 0;
};

Status compute_c_shape(const Dims &a, const Dims &b, bool trans_lhs, bool trans_rhs, bool trans_out, Dims *out);
Status resolve_spec(const rt_matmul_desc &desc, Spec *spec);
void fill_public_spec(const Spec &s, rt_gemm_spec *out);

} // namespace rt
