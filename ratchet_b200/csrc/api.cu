// C ABI of the library: device, storage, plan ("compile") and launch ("dispatch").
// Stands where ratchet-core's device / storage / compiled-op layers stand
// (crates/ratchet-core/src/gpu/device.rs, storage/gpu_buffer.rs, op.rs:304-362, compiled_op.rs,
// executable.rs:25-54 of the reference).
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "arena.hpp"
#include "kernels.hpp"
#include "ratchet_b200.h"
#include "spec.hpp"

namespace rt {
Status dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int *n);
Status quantize_q8_0(const float *x, uint64_t numel, rt_dtype dt, uint8_t *out);
Status dequantize_q8_0(const uint8_t *src, uint64_t numel, rt_dtype dt, float *out);
Status transcode_gguf_q8_0(const uint8_t *blocks, uint64_t n_blocks, rt_dtype dt, uint8_t *out);
Status quantize_q4_k(const float *x, uint64_t numel, uint8_t *out);
Status dequantize_q4_k(const uint8_t *src, uint64_t numel, float *out);
} // namespace rt

using namespace rt;

// Device memory is recycled through size-class free lists, the role of the reference's buffer
// pool (crates/ratchet-core/src/gpu/pools/buffer_pool.rs:97-119): a freed buffer is kept and
// handed to the next request of the same class, so steady-state steps call neither cudaMalloc nor
// cudaFree (which would serialise the device).
struct rt_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    std::mutex pool_mu;
    std::unordered_map<uint64_t, std::vector<void *>> pool; // size class -> free blocks
    uint64_t pooled_bytes = 0;
    // compiled-op cache: one plan per distinct node description (the role of the reference's KernelKey lookup,
    // crates/ratchet-core/src/ops/matmul.rs:485-524 and op.rs:169-196)
    std::mutex plan_mu;
    std::unordered_map<std::string, rt_plan *> plans;
    std::mutex kept_mu;
    std::unordered_map<const void *, int> kept_ptrs; // weight pointers some plan keeps a dequantised copy of
};

static inline uint64_t size_class(uint64_t n) {
    if (n <= 4096) return (n + 255) / 256 * 256;
    uint64_t c = 4096;
    while (c < n) c <<= 1;
    // quarter steps between powers of two bound the slack at 25 %
    uint64_t q = c / 8;
    uint64_t r = c / 2 + (n - c / 2 + q - 1) / q * q;
    return r < c ? r : c;
}

struct rt_buffer {
    rt_device *dev = nullptr;
    void *ptr = nullptr;
    uint64_t size = 0;  // bytes the caller may use
    uint64_t klass = 0; // bytes allocated
};

enum PlanKernel { PK_GEMM_SIMT, PK_GEMV_SIMT, PK_ROWVEC_MAT, PK_Q8_GEMV_MMA, PK_Q8_GEMV_UMMA, PK_Q4K_GEMV, PK_Q4K_GEMV_UMMA, PK_GEMM_UMMA };

struct rt_plan {
    rt_device *dev = nullptr;
    Spec spec;
    PlanKernel kernel = PK_GEMM_SIMT;
    std::string name;
    int launches = 1;
    int split = 1;
    int nv = 1;
    GemvUmmaConfig gemv_umma{};
    Q4kUmmaConfig q4k_umma{};
    int nv2 = 0;           // streaming Q8_0 kernel: vectors beyond the first launch's 8, taken 8 at a time (9..24 in all)
    bool chain_ok = false; // a Q8_0H x f16 GEMV the persistent chain kernel can take as a node
    MatmulParams params{}; // everything but the pointers
    uint64_t lhs_scale_offset = 0;
    // tensor-core GEMM: operand roles, tile width, and the scratch that holds dequantised weights
    bool lhs_is_q = false; // the lhs is the kernel's Q operand (trans_out), else its P operand
    int R = 0, S = 0, u_stacks = 1, p_stack = 1, q_stack = 1, bn = 128;
    bool tf32x3 = false;   // dense f32 on the tensor cores: three TF32 MMAs per product
    bool rhs_transpose = false; // rhs is stored [K][N]: transposed into act_scratch ahead of the GEMM
    int k_pad = 0;              // with rhs_transpose, 16-bit: K rounded up to a multiple of 8 when it is not one
                                // (lhs rows are then copied, zero-padded, into `scratch`); 0 = K as it is
    void *scratch = nullptr;     // dequantised weights (f16)
    uint64_t scratch_bytes = 0;
    void *act_scratch = nullptr; // bf16 activations cast to f16 (quantised weights only)
    uint64_t act_scratch_bytes = 0;
    uint64_t act_scale_off = 0; // bf16 cast: where the per-row factors (f32) start inside act_scratch
    void *wdq = nullptr;         // f32 GEMM over Q8_0F weights: the weights as f32 ((i8)q * d, quant.rs:114-120)
    uint64_t wdq_bytes = 0;
    // RT_EPILOGUE_SILU_MUL on a route that does not fold the gate/up pairs itself: the plain node's [.., 2*ff] output
    // goes here and an elementwise launch writes the [.., ff] result
    bool pair = false;
    void *pair_scratch = nullptr;
    uint64_t pair_bytes = 0;
    int refs = 1;                // holders: the device's cache and every rt_matmul_plan call that returned this plan
    std::string key;             // its entry in the device's cache
    // Dequantised copies of weights the caller flagged RT_LAUNCH_LHS_CONSTANT, by weight pointer: the pre-pass then
    // runs once per weight instead of once per launch, and plans shared by many same-shaped layers do not share scratch.
    std::mutex weights_mu;
    std::unordered_map<const void *, void *> kept_weights;
    ~rt_plan() {
        if (scratch || act_scratch || pair_scratch || wdq || !kept_weights.empty()) cudaSetDevice(dev->ordinal);
        if (wdq) cudaFree(wdq);
        if (scratch) cudaFree(scratch);
        if (act_scratch) cudaFree(act_scratch);
        if (pair_scratch) cudaFree(pair_scratch);
        for (auto &kv : kept_weights) cudaFree(kv.second);
    }
};

// Everything of a node description that routing looks at, field by field (the struct has padding bytes), plus the
// debugging switches that change routing.
static std::string plan_key(const rt_matmul_desc &d) {
    std::string k;
    auto put = [&k](long long v) { k.append(reinterpret_cast<const char *>(&v), sizeof(v)); };
    auto put_shape = [&](const rt_shape &s) {
        put(s.rank);
        for (int i = 0; i < s.rank && i < RT_MAX_RANK; i++) put(s.dims[i]);
    };
    put(d.lhs_dt); put(d.rhs_dt); put(d.has_bias ? d.bias_dt : -1);
    put_shape(d.lhs_shape); put_shape(d.rhs_shape);
    if (d.has_bias) put_shape(d.bias_shape);
    put(d.has_bias != 0); put(d.trans_lhs != 0); put(d.trans_rhs != 0); put(d.trans_out != 0); put(d.epilogue);
    for (const char *name : {"RT_FORCE_KERNEL", "RT_GEMV_UMMA", "RT_Q4K_UMMA", "RT_GEMM_PAIR", "RT_GEMM_PAIR_MIN", "RT_TF32_BN", "RT_TF32_PRESPLIT", "RT_Q4K_WALK_FROM", "RT_KEEP_WEIGHTS"}) {
        const char *v = getenv(name);
        k += '|';
        if (v) k += v;
    }
    return k;
}

// Scratch areas that take the place of a plan's own during one launch.
struct ScratchSet {
    void *scratch = nullptr, *act = nullptr, *pair = nullptr, *wdq = nullptr;
};

struct rt_executable {
    rt_device *dev = nullptr;
    std::vector<rt_dispatch> nodes;
    // One allocation for every intermediate tensor and every node's plan scratch, placed by the activation planner
    // (arena.cpp, the reference's BufferAllocator::greedy_by_size).
    std::vector<ScratchSet> scratch; // per node: where its plan's scratch areas live in the arena
    std::vector<void *> tensors;     // per intermediate: its address in the arena
    void *arena = nullptr;
    uint64_t arena_bytes = 0, record_bytes = 0;
    int n_objects = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    GemvChain *chain = nullptr; // the whole node list as one persistent kernel (gemv_q8_chain.cu)
    bool chain_refused = false; // its launch was refused once: dispatch node by node from then on
    std::string how = "nodes";
    int launches = 0;
    ~rt_executable() { // also what a failed rt_executable_create leaves behind
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
        if (chain) gemv_chain_destroy(chain);
        if (arena) {
            cudaSetDevice(dev->ordinal);
            cudaFree(arena);
        }
    }
};

// RT_KEEP_WEIGHTS=0: dequantise on every launch even for weights flagged constant (A/B timing, memory-tight callers).
static bool keep_weights_enabled() {
    const char *v = getenv("RT_KEEP_WEIGHTS");
    return !(v && v[0] == '0');
}

// The dequantised copy the plan keeps of a constant weight, by weight pointer; *filled says whether an earlier
// launch already wrote it.  A new weight gets its copy here unless the stream is capturing or memory is short
// (nullptr: the caller uses scratch).
static void *kept_weight_copy(rt_plan *plan, const void *lhs, cudaStream_t st, bool *filled, uint64_t bytes) {
    *filled = false;
    if (!keep_weights_enabled()) return nullptr;
    std::lock_guard<std::mutex> lk(plan->weights_mu);
    auto it = plan->kept_weights.find(lhs);
    if (it != plan->kept_weights.end()) {
        *filled = true;
        return it->second;
    }
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    void *kept = nullptr;
    if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone &&
        cudaMalloc(&kept, bytes) == cudaSuccess) {
        plan->kept_weights.emplace(lhs, kept);
        std::lock_guard<std::mutex> dl(plan->dev->kept_mu);
        plan->dev->kept_ptrs[lhs]++;
        return kept;
    }
    cudaGetLastError(); // no room, or capturing
    return nullptr;
}

static rt_status launch_node(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream,
                             const rt_launch_opts *opts, const ScratchSet *ov);

#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (expr);                                                                   \
        if (e__ != cudaSuccess)                                                                     \
            return fail(RT_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__));          \
    } while (0)

extern "C" {

const char *rt_last_error(void) { return last_error().c_str(); }

const char *rt_status_name(rt_status s) {
    switch (s) {
    case RT_OK: return "RT_OK";
    case RT_ERR_SHAPE: return "RT_ERR_SHAPE";
    case RT_ERR_DTYPE: return "RT_ERR_DTYPE";
    case RT_ERR_INVARIANT: return "RT_ERR_INVARIANT";
    case RT_ERR_ARG: return "RT_ERR_ARG";
    case RT_ERR_CUDA: return "RT_ERR_CUDA";
    case RT_ERR_UNSUPPORTED: return "RT_ERR_UNSUPPORTED";
    case RT_ERR_NOMEM: return "RT_ERR_NOMEM";
    case RT_ERR_COMM: return "RT_ERR_COMM";
    case RT_ERR_COMM_TIMEOUT: return "RT_ERR_COMM_TIMEOUT";
    }
    return "RT_ERR_?";
}

const char *rt_version(void) { return "ratchet_b200 0.1.0 sm_100a"; }

/* ------------------------------------------------------------------ dtypes and layouts */

size_t rt_dtype_size(rt_dtype dt) { return dtype_valid(dt) ? dtype_size(dt) : 0; }
int32_t rt_dtype_is_quantized(rt_dtype dt) { return dtype_valid(dt) && is_quantized(dt) ? 1 : 0; }

rt_status rt_dtype_activation(rt_dtype dt, rt_dtype *out) {
    if (!out || !dtype_valid(dt)) return fail(RT_ERR_ARG, "rt_dtype_activation: bad argument");
    *out = activation_dt(dt);
    return RT_OK;
}

rt_status rt_dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int32_t *n_segs) {
    if (!segs || !n_segs || !dtype_valid(dt)) return fail(RT_ERR_ARG, "rt_dtype_segments: bad argument");
    rt_segment tmp[2];
    int n = 0;
    Status st = dtype_segments(dt, numel, tmp, &n);
    if (!st.ok()) return fail(st);
    if (*n_segs < n) return fail(RT_ERR_ARG, "rt_dtype_segments: segment array too small");
    for (int i = 0; i < n; i++) segs[i] = tmp[i];
    *n_segs = n;
    return RT_OK;
}

rt_status rt_dtype_nbytes(rt_dtype dt, uint64_t numel, uint64_t *nbytes) {
    if (!nbytes || !dtype_valid(dt)) return fail(RT_ERR_ARG, "rt_dtype_nbytes: bad argument");
    rt_segment tmp[2];
    int n = 0;
    Status st = dtype_segments(dt, numel, tmp, &n);
    if (!st.ok()) return fail(st);
    uint64_t total = 0;
    for (int i = 0; i < n; i++) total += tmp[i].size;
    *nbytes = total;
    return RT_OK;
}

rt_status rt_quantize_q8_0(const float *src, uint64_t numel, rt_dtype dt, void *out) {
    if (!src || !out || (dt != RT_Q8_0H && dt != RT_Q8_0F)) return fail(RT_ERR_ARG, "rt_quantize_q8_0: bad argument");
    Status st = quantize_q8_0(src, numel, dt, (uint8_t *)out);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_dequantize_q8_0(const void *src, uint64_t numel, rt_dtype dt, float *out) {
    if (!src || !out || (dt != RT_Q8_0H && dt != RT_Q8_0F)) return fail(RT_ERR_ARG, "rt_dequantize_q8_0: bad argument");
    Status st = dequantize_q8_0((const uint8_t *)src, numel, dt, out);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_transcode_gguf_q8_0(const void *blocks, uint64_t n_blocks, rt_dtype dt, void *out) {
    if (!blocks || !out || (dt != RT_Q8_0H && dt != RT_Q8_0F))
        return fail(RT_ERR_ARG, "rt_transcode_gguf_q8_0: bad argument");
    Status st = transcode_gguf_q8_0((const uint8_t *)blocks, n_blocks, dt, (uint8_t *)out);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_quantize_q4_k(const float *src, uint64_t numel, void *out) {
    if (!src || !out) return fail(RT_ERR_ARG, "rt_quantize_q4_k: bad argument");
    Status st = quantize_q4_k(src, numel, (uint8_t *)out);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_dequantize_q4_k(const void *src, uint64_t numel, float *out) {
    if (!src || !out) return fail(RT_ERR_ARG, "rt_dequantize_q4_k: bad argument");
    Status st = dequantize_q4_k((const uint8_t *)src, numel, out);
    return st.ok() ? RT_OK : fail(st);
}

/* ------------------------------------------------------------------ Matmul rules */

rt_status rt_matmul_spec(const rt_matmul_desc *desc, rt_gemm_spec *spec) {
    if (!desc || !spec) return fail(RT_ERR_ARG, "rt_matmul_spec: null argument");
    Spec s;
    Status st = resolve_spec(*desc, &s);
    if (!st.ok()) return fail(st);
    fill_public_spec(s, spec);
    return RT_OK;
}

rt_status rt_matmul_out_shape(const rt_matmul_desc *desc, rt_shape *out) {
    if (!desc || !out) return fail(RT_ERR_ARG, "rt_matmul_out_shape: null argument");
    if (desc->lhs_shape.rank < 0 || desc->lhs_shape.rank > RT_MAX_RANK || desc->rhs_shape.rank < 0 ||
        desc->rhs_shape.rank > RT_MAX_RANK)
        return fail(RT_ERR_ARG, "rank out of range");
    Dims c;
    Status st = compute_c_shape(to_dims(desc->lhs_shape), to_dims(desc->rhs_shape), desc->trans_lhs != 0,
                                desc->trans_rhs != 0, desc->trans_out != 0, &c);
    if (!st.ok()) return fail(st);
    if (desc->epilogue == RT_EPILOGUE_SILU_MUL && !c.empty()) c.back() /= 2; // gate | up folded (see resolve_spec for the checks)
    if (!from_dims(c, out)) return fail(RT_ERR_SHAPE, "output rank exceeds RT_MAX_RANK");
    return RT_OK;
}

/* ------------------------------------------------------------------ device and storage */

rt_status rt_device_create(int32_t ordinal, rt_device **dev) {
    if (!dev) return fail(RT_ERR_ARG, "rt_device_create: null argument");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(RT_ERR_CUDA, std::string("no CUDA device: this library has no CPU path (") +
                                     (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0") + ")");
    if (ordinal < 0 || ordinal >= count) return fail(RT_ERR_ARG, "rt_device_create: ordinal out of range");
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(RT_ERR_UNSUPPORTED, std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) +
                                            std::to_string(prop.minor) + "; the kernels are built for sm_100a only");
    CUDA_TRY(cudaSetDevice(ordinal));
    rt_device *d = new (std::nothrow) rt_device();
    if (!d) return fail(RT_ERR_NOMEM, "out of host memory");
    d->ordinal = ordinal;
    d->sm_count = prop.multiProcessorCount;
    d->cc_major = prop.major;
    d->cc_minor = prop.minor;
    e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete d;
        return fail(RT_ERR_CUDA, std::string("cudaStreamCreate: ") + cudaGetErrorString(e));
    }
    *dev = d;
    return RT_OK;
}

rt_status rt_device_destroy(rt_device *dev) {
    if (!dev) return RT_OK;
    cudaSetDevice(dev->ordinal);
    if (dev->stream) cudaStreamSynchronize(dev->stream);
    for (auto &kv : dev->plans)
        if (--kv.second->refs <= 0) delete kv.second;
    dev->plans.clear();
    for (auto &kv : dev->pool)
        for (void *p : kv.second) cudaFree(p);
    if (dev->stream) cudaStreamDestroy(dev->stream);
    delete dev;
    return RT_OK;
}

rt_status rt_device_sync(rt_device *dev) {
    if (!dev) return fail(RT_ERR_ARG, "rt_device_sync: null device");
    CUDA_TRY(cudaSetDevice(dev->ordinal));
    CUDA_TRY(cudaStreamSynchronize(dev->stream));
    int site = 0;
    CUDA_TRY(umma_take_error(&site, dev->stream));
    if (site != 0)
        return fail(RT_ERR_CUDA, "a tensor-core GEMM gave up a bounded wait (site " + std::to_string(site) +
                                     "): its output is incomplete");
    CUDA_TRY(umma_tf32_take_error(&site, dev->stream));
    if (site != 0)
        return fail(RT_ERR_CUDA, "an f32 tensor-core GEMM gave up a bounded wait (site " + std::to_string(site) + "): its output is incomplete");
    CUDA_TRY(gemv_umma_take_error(&site, dev->stream));
    if (site != 0)
        return fail(RT_ERR_CUDA, "a tensor-memory GEMV gave up a bounded wait (site " + std::to_string(site) + "): its output is incomplete");
    CUDA_TRY(gemv_chain_take_error(&site, dev->stream));
    if (site != 0)
        return fail(RT_ERR_CUDA, "a GEMV chain gave up a bounded wait (site " + std::to_string(site) + "): its outputs are incomplete");
    CUDA_TRY(gemv_q4k_take_error(&site, dev->stream));
    if (site != 0) return fail(RT_ERR_CUDA, "a Q4_K GEMV gave up waiting for its weight copies: its output is incomplete");
    CUDA_TRY(gemv_q4k_umma_take_error(&site, dev->stream));
    if (site != 0)
        return fail(RT_ERR_CUDA, "a tensor-memory Q4_K GEMV gave up a bounded wait (site " + std::to_string(site) + "): its output is incomplete");
    CUDA_TRY(gemv_take_error(&site, dev->stream));
    if (site != 0) return fail(RT_ERR_CUDA, "a GEMV gave up waiting for its weight copies: its output is incomplete");
    return RT_OK;
}

void *rt_device_stream(rt_device *dev) { return dev ? (void *)dev->stream : nullptr; }
int32_t rt_device_sm_count(rt_device *dev) { return dev ? dev->sm_count : 0; }
int32_t rt_device_ordinal(rt_device *dev) { return dev ? dev->ordinal : -1; }

rt_status rt_buffer_alloc(rt_device *dev, uint64_t nbytes, rt_buffer **buf) {
    if (!dev || !buf) return fail(RT_ERR_ARG, "rt_buffer_alloc: null argument");
    uint64_t size = nbytes < 16 ? 16 : (nbytes + 3) / 4 * 4; // buffer_pool.rs:82-95
    uint64_t klass = size_class(size);
    void *p = nullptr;
    {
        std::lock_guard<std::mutex> lk(dev->pool_mu);
        auto it = dev->pool.find(klass);
        if (it != dev->pool.end() && !it->second.empty()) {
            p = it->second.back();
            it->second.pop_back();
            dev->pooled_bytes -= klass;
        }
    }
    if (!p) {
        CUDA_TRY(cudaSetDevice(dev->ordinal));
        cudaError_t e = cudaMalloc(&p, klass);
        if (e == cudaErrorMemoryAllocation) {
            // give the pooled blocks back and retry once
            cudaGetLastError();
            std::lock_guard<std::mutex> lk(dev->pool_mu);
            for (auto &kv : dev->pool) {
                for (void *q : kv.second) cudaFree(q);
                kv.second.clear();
            }
            dev->pooled_bytes = 0;
            e = cudaMalloc(&p, klass);
        }
        if (e != cudaSuccess)
            return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA, std::string("cudaMalloc: ") + cudaGetErrorString(e));
    }
    rt_buffer *b = new (std::nothrow) rt_buffer();
    if (!b) {
        cudaFree(p);
        return fail(RT_ERR_NOMEM, "out of host memory");
    }
    b->dev = dev;
    b->ptr = p;
    b->size = size;
    b->klass = klass;
    *buf = b;
    return RT_OK;
}

// A freed block may be handed out again at once: work already queued on the device's stream that
// still uses it runs before anything a later owner queues on that stream.
rt_status rt_buffer_free(rt_buffer *buf) {
    if (!buf) return RT_OK;
    rt_device *dev = buf->dev;
    {
        // a weight that goes away takes the dequantised copies plans keep of it along: the block may come back
        // from the pool holding another tensor
        bool kept = false;
        {
            std::lock_guard<std::mutex> lk(dev->kept_mu);
            kept = dev->kept_ptrs.erase(buf->ptr) > 0;
        }
        if (kept) {
            cudaSetDevice(dev->ordinal);
            std::lock_guard<std::mutex> lk(dev->plan_mu);
            for (auto &kv : dev->plans) {
                std::lock_guard<std::mutex> wl(kv.second->weights_mu);
                auto it = kv.second->kept_weights.find(buf->ptr);
                if (it != kv.second->kept_weights.end()) {
                    cudaFree(it->second);
                    kv.second->kept_weights.erase(it);
                }
            }
        }
    }
    {
        std::lock_guard<std::mutex> lk(dev->pool_mu);
        dev->pool[buf->klass].push_back(buf->ptr);
        dev->pooled_bytes += buf->klass;
    }
    delete buf;
    return RT_OK;
}

void *rt_buffer_ptr(rt_buffer *buf) { return buf ? buf->ptr : nullptr; }
uint64_t rt_buffer_size(rt_buffer *buf) { return buf ? buf->size : 0; }

rt_status rt_upload(rt_device *dev, rt_buffer *dst, uint64_t dst_off, const void *host, uint64_t n, int32_t sync) {
    if (!dev || !dst || (!host && n)) return fail(RT_ERR_ARG, "rt_upload: null argument");
    if (dst_off > dst->size || n > dst->size - dst_off) return fail(RT_ERR_ARG, "rt_upload: range exceeds the buffer");
    CUDA_TRY(cudaSetDevice(dev->ordinal));
    if (n) CUDA_TRY(cudaMemcpyAsync((char *)dst->ptr + dst_off, host, n, cudaMemcpyHostToDevice, dev->stream));
    if (sync) CUDA_TRY(cudaStreamSynchronize(dev->stream));
    return RT_OK;
}

rt_status rt_download(rt_device *dev, const rt_buffer *src, uint64_t src_off, void *host, uint64_t n, int32_t sync) {
    if (!dev || !src || (!host && n)) return fail(RT_ERR_ARG, "rt_download: null argument");
    if (src_off > src->size || n > src->size - src_off) return fail(RT_ERR_ARG, "rt_download: range exceeds the buffer");
    CUDA_TRY(cudaSetDevice(dev->ordinal));
    if (n) CUDA_TRY(cudaMemcpyAsync(host, (const char *)src->ptr + src_off, n, cudaMemcpyDeviceToHost, dev->stream));
    if (sync) CUDA_TRY(cudaStreamSynchronize(dev->stream));
    return RT_OK;
}

rt_status rt_host_alloc(uint64_t nbytes, void **ptr) {
    if (!ptr) return fail(RT_ERR_ARG, "rt_host_alloc: null argument");
    CUDA_TRY(cudaMallocHost(ptr, nbytes ? nbytes : 1));
    return RT_OK;
}

rt_status rt_host_free(void *ptr) {
    if (!ptr) return RT_OK;
    CUDA_TRY(cudaFreeHost(ptr));
    return RT_OK;
}

/* ------------------------------------------------------------------ compile + dispatch */

// RT_GEMV_CHAIN=0 keeps executables on one launch per node (a debugging and A/B timing switch).
static bool chain_enabled() {
    const char *v = getenv("RT_GEMV_CHAIN");
    return !(v && v[0] == '0');
}

// RT_FORCE_KERNEL=simt keeps every node on the CUDA-core kernels (a debugging switch in the
// spirit of the reference's RATCHET_* variables, gpu/device.rs:92-99).

// RT_Q4K_UMMA=1 sends large Q4_K GEMVs through tensor memory (gemv_q4k_umma.cu).  Off by default: measured on
// [8192,3072] it is faster than the warp-MMA kernel only with two vectors (10.1 against 11.1 us; 9.0 against 8.3 us with
// one, 26 against 17 us with sixteen): unpacking nibbles to int8 codes moves 5.5 bytes through shared memory per weight
// byte, and a CTA that needs the SM to itself cannot overlap the next launch's prologue with this one's tail.
static bool q4k_umma_enabled() {
    const char *v = getenv("RT_Q4K_UMMA");
    return v && v[0] == '1';
}

// RT_GEMM_PAIR=0 keeps the tensor-core GEMM on one CTA per tile (A/B timing).
static bool gemm_pair_enabled() {
    const char *v = getenv("RT_GEMM_PAIR");
    return !(v && v[0] == '0');
}

// fewest 256 x 256 tiles at which the CTA-pair kernel is taken (RT_GEMM_PAIR_MIN overrides: A/B timing)
static long long gemm_pair_min_tiles(int sm_count) {
    const char *v = getenv("RT_GEMM_PAIR_MIN");
    // from four fifths of a wave of pairs (measured: 64 tiles on 74 pairs, Q4_K [8192,3072] x 512 rows: 27.2 -> 25.1 us;
    // 36 tiles, the Whisper MLP: 22.7 -> 30.9 us)
    return v ? atoll(v) : (long long)(sm_count / 2) * 4 / 5;
}

static bool force_simt() {
    const char *v = getenv("RT_FORCE_KERNEL");
    return v && std::string(v) == "simt";
}

// The tensor-core GEMM takes nn::Linear-shaped nodes: both operands K-major, 16-bit activations.
// The tensor-core GEMMs take both operands K-major: op(lhs) [M][K] as stored, and op(rhs) as [N][K], which
// is how trans_rhs stores it (the Linear form).  A dense rhs stored [K][N] (the attention products
// q.kT and softmax.v of the models, rank 4, no transposes) is made K-major by a transposing pass first.
static bool umma_eligible(const rt_matmul_desc &d, const Spec &s) {
    if (force_simt()) return false;
    if (s.trans_lhs) return false;
    if (!s.trans_rhs) {
        if (d.lhs_dt != d.rhs_dt || s.trans_out) return false;
        // f32: only where the GEMM's vector stores apply (output rows of whole 16-byte groups) and not
        // below 16 rows, where three launches cost more than the CUDA-core kernel
        if (d.rhs_dt == RT_F32 && s.N % 4 != 0) return false;
        if (d.rhs_dt == RT_F32 && s.M < 16) return false;
    }
    if (d.rhs_dt == RT_F32) {
        // dense f32, or the reference's default pair (Q8_0F, F32) in the Linear form with the weights dequantised to f32
        if ((d.lhs_dt != RT_F32 && d.lhs_dt != RT_Q8_0F) || !umma_tf32_supported(s.K)) return false;
    } else {
        if (d.rhs_dt != RT_F16 && d.rhs_dt != RT_BF16) return false;
        const bool dense = d.lhs_dt == d.rhs_dt;
        if (!dense && d.lhs_dt != RT_Q8_0H && d.lhs_dt != RT_Q4_K) return false;
        // a dense 16-bit product with rhs [K][N] whose K is not a multiple of 8 (Whisper's softmax.v, K = 1500):
        // both operands are repacked anyway or cheaply, with K zero-padded to the next multiple of 8
        const long long k_eff = (!s.trans_rhs && dense) ? (s.K + 7) / 8 * 8 : s.K;
        if (!umma_gemm_supported(k_eff)) return false;
    }
    if (s.M < 1 || s.N < 9 || s.stacks < 1) return false; // up to 8 columns: the streaming GEMV kernels
    if ((double)s.M * (double)s.N * (double)s.K * (double)s.stacks < (double)(1 << 21)) return false;
    return true;
}

static rt_status build_plan(rt_device *dev, const rt_matmul_desc *desc, rt_plan **plan);

rt_status rt_matmul_plan(rt_device *dev, const rt_matmul_desc *desc, rt_plan **plan) {
    if (!dev || !desc || !plan) return fail(RT_ERR_ARG, "rt_matmul_plan: null argument");
    if (desc->lhs_shape.rank < 0 || desc->lhs_shape.rank > RT_MAX_RANK || desc->rhs_shape.rank < 0 || desc->rhs_shape.rank > RT_MAX_RANK ||
        (desc->has_bias && (desc->bias_shape.rank < 0 || desc->bias_shape.rank > RT_MAX_RANK)))
        return fail(RT_ERR_ARG, "rank out of range");
    const std::string key = plan_key(*desc);
    std::lock_guard<std::mutex> lk(dev->plan_mu); // one plan is built at a time per device: equal descriptions share it
    auto it = dev->plans.find(key);
    if (it != dev->plans.end()) {
        it->second->refs++;
        *plan = it->second;
        return RT_OK;
    }
    rt_plan *pl = nullptr;
    rt_status st = build_plan(dev, desc, &pl);
    if (st != RT_OK) return st;
    pl->key = key;
    pl->refs = 2; // the cache and the caller
    dev->plans.emplace(key, pl);
    *plan = pl;
    return RT_OK;
}

static rt_status build_plan(rt_device *dev, const rt_matmul_desc *desc, rt_plan **plan) {
    rt_plan *pl = new (std::nothrow) rt_plan();
    if (!pl) return fail(RT_ERR_NOMEM, "out of host memory");
    Status st = resolve_spec(*desc, &pl->spec);
    if (!st.ok()) {
        delete pl;
        return fail(st);
    }
    const Spec &s = pl->spec;
    pl->dev = dev;
    MatmulParams &p = pl->params;
    p.M = (int)s.M; p.N = (int)s.N; p.K = (int)s.K;
    p.stacks = (int)s.stacks; p.lhs_stack = (int)s.lhs_stack; p.rhs_stack = (int)s.rhs_stack;
    p.trans_lhs = s.trans_lhs; p.trans_rhs = s.trans_rhs; p.trans_out = s.trans_out;
    p.bias_mode = BIAS_NONE;
    if (s.has_bias) {
        if (s.trans_out) p.bias_mode = BIAS_PER_M;
        else if (s.N == 1 && !s.trans_lhs && s.bias_len == s.M && s.M != 1) p.bias_mode = BIAS_PER_M; // gemv.rs:476-490
        else p.bias_mode = BIAS_PER_N;
    }
    p.bias_dt = s.has_bias ? desc->bias_dt : RT_F32;
    p.epilogue = s.epilogue;
    p.lhs_batch_elems = s.M * s.K;
    p.lhs_batch_scale_bytes = 0;
    pl->lhs_scale_offset = 0;
    if (desc->lhs_dt == RT_Q8_0H || desc->lhs_dt == RT_Q8_0F) {
        rt_segment seg[2];
        int n = 0;
        st = dtype_segments(desc->lhs_dt, (uint64_t)(s.lhs_stack * s.M * s.K), seg, &n);
        if (!st.ok()) {
            delete pl;
            return fail(st);
        }
        pl->lhs_scale_offset = seg[1].offset;
        p.lhs_batch_scale_bytes = s.M * s.K / 32 * (desc->lhs_dt == RT_Q8_0H ? 2 : 4);
    }

    // Routing (ops/matmul.rs:540-592 picks GEMV when rhs is a vector; here "skinny" nodes, where
    // the weight bytes dominate, also take the streaming kernel).
    const bool q8 = desc->lhs_dt == RT_Q8_0H || desc->lhs_dt == RT_Q8_0F;
    const bool empty = s.M == 0 || s.N == 0 || s.stacks == 0;
    const int gemv_split = (q8 && s.K > 0 && !empty && !force_simt())
                               ? q8_gemv_mma_pick_split(p.M, p.K, dev->sm_count, desc->lhs_dt == RT_Q8_0H ? 2 : 4) : 0;
    // short rows against very many of them (the Whisper logits, [51865, 384]): the 16-row CTAs of the streaming
    // kernel come to 3,242 tiny CTAs; the CUDA-core GEMV with 8 rows per warp is faster there (12.6 against 16.4 us)
    const bool short_rows = q8 && s.N == 1 && s.K <= 512 && s.M >= 16384 && s.K % 32 == 0;
    if (gemv_split > 0 && !short_rows && desc->rhs_dt == RT_F16 && !s.trans_lhs && s.N >= 1 && s.N <= 8 && (s.N == 1 || s.trans_rhs) && s.K > 0 && !empty) {
        pl->nv = (int)s.N;
        pl->split = gemv_split;
        // one vector against f16-scaled Q8_0 at a size that fills the machine: the tensor-memory GEMV
        const char *env_gu = getenv("RT_GEMV_UMMA");
        pl->chain_ok = !(env_gu && env_gu[0] == '0') && desc->lhs_dt == RT_Q8_0H && s.N == 1 && s.stacks == 1 &&
                       s.lhs_stack == 1 && s.rhs_stack == 1 &&
                       q8_gemv_umma_config(p.M, p.K, dev->sm_count, &pl->gemv_umma) && pl->gemv_umma.rb >= 8;
        // launched on its own, the tensor-memory kernel only pays from about 22 rows per CTA: below that its
        // fixed cost (tensor-memory allocation, digits of x, the MMA pipeline's depth) outweighs the streaming
        // kernel's (measured on [2560,2560]: 13.2 us against 5.2 us; equal at [3072,3072]; 7.1 against 10.4 us
        // at [4096,4096])
        const bool umma_ok = pl->chain_ok && pl->gemv_umma.rb >= 22;
        pl->kernel = umma_ok ? PK_Q8_GEMV_UMMA : PK_Q8_GEMV_MMA;
        if (umma_ok)
            pl->name = std::string("q8_gemv_umma_h_rb") + std::to_string(pl->gemv_umma.rb) + "_split" +
                       std::to_string(pl->gemv_umma.split) + "_ring" + std::to_string(pl->gemv_umma.ring);
        else
        pl->name = std::string("q8_gemv_mma_") + (desc->lhs_dt == RT_Q8_0H ? "h" : "f") + "_nv" + std::to_string(pl->nv) +
                   "_split" + std::to_string(pl->split);
    } else if (gemv_split > 0 && desc->rhs_dt == RT_F16 && !s.trans_lhs && s.trans_rhs && s.trans_out && s.N >= 9 && s.N <= 24 &&
               s.stacks == 1 && s.K > 0 && !empty &&
               // two passes over weights of 32 Mi values or more cost more than the tensor-core GEMM even when that has to
               // dequantise first ([16384,3072] x 17..24 rows: 52 .. 55 us against 24 us with a kept f16 copy, ~50 without)
               !(s.N > 16 && (double)s.M * (double)s.K >= (double)(1 << 25) && umma_eligible(*desc, s))) {
        // 9..24 vectors against Q8_0: the streaming kernel with two groups of eight MMA columns takes up to 16 in one
        // pass over the weights; 17..24 are a pass of 16 and a pass of the rest (the weights are read again, from L2
        // where they fit), which still is under the dequantise + tensor-core GEMM route; with trans_out each
        // vector's outputs are contiguous, so a later pass is the same problem on offset pointers.
        pl->kernel = PK_Q8_GEMV_MMA;
        pl->nv = (int)std::min<int64_t>(s.N, 16);
        pl->nv2 = (int)s.N - pl->nv;
        pl->split = gemv_split;
        pl->launches = 1 + (pl->nv2 > 0 ? 1 : 0);
        pl->name = std::string("q8_gemv_mma_") + (desc->lhs_dt == RT_Q8_0H ? "h" : "f") + "_nv" + std::to_string(pl->nv) +
                   (pl->nv2 ? "+" + std::to_string(pl->nv2) : std::string()) + "_split" + std::to_string(pl->split);
    } else if (desc->lhs_dt == RT_Q4_K && desc->rhs_dt == RT_F16 && !s.trans_lhs && s.N >= 1 && s.N <= 16 &&
               (s.N == 1 || s.trans_rhs) && !empty && !force_simt() && s.stacks == 1 && q4k_umma_enabled() &&
               (double)s.M * (double)s.K >= (double)(1 << 22) &&
               q4k_gemv_umma_config(p.M, p.K, (int)s.N, dev->sm_count, &pl->q4k_umma)) {
        // weights of a size that fills the machine: nibbles to int8 codes in shared memory, sums on the tensor cores
        pl->kernel = PK_Q4K_GEMV_UMMA;
        pl->nv = (int)s.N;
        const Q4kUmmaConfig &c = pl->q4k_umma;
        pl->name = std::string("q4k_gemv_umma_nv") + std::to_string(pl->nv) + "_rb" + std::to_string(c.rb) + "_split" + std::to_string(c.split) +
                   "_ring" + std::to_string(c.raw_ring) + "x" + std::to_string(c.a_ring);
    } else if (desc->lhs_dt == RT_Q4_K && desc->rhs_dt == RT_F16 && !s.trans_lhs && s.N >= 1 && s.N <= 16 &&
               (s.N == 1 || s.trans_rhs) && !empty && !force_simt() &&
               q4k_gemv_pick_split(p.M, p.K, (int)s.N, (int)s.stacks, dev->sm_count) > 0) {
        pl->kernel = PK_Q4K_GEMV;
        pl->nv = (int)s.N;
        pl->split = q4k_gemv_pick_split(p.M, p.K, (int)s.N, (int)s.stacks, dev->sm_count); // split | groups per CTA << 8 | buffers << 16
        pl->name = std::string("q4k_gemv_mma_nv") + std::to_string(pl->nv) + "_split" + std::to_string(pl->split & 0xff) +
                   (((pl->split >> 8) & 0xff) > 1 ? "_walk" + std::to_string((pl->split >> 8) & 0xff) + "x" + std::to_string((pl->split >> 16) & 0xff) + "buf"
                                                   : std::string());
    } else if (s.M == 1 && s.N >= 2 && !s.trans_lhs && !s.trans_rhs && desc->lhs_dt == desc->rhs_dt && !is_quantized(desc->lhs_dt) &&
               (desc->rhs_dt == RT_F32 || desc->rhs_dt == RT_F16 || desc->rhs_dt == RT_BF16) && !empty && !force_simt() &&
               s.stacks <= 65535) {
        // one row against a dense [K][N] matrix (q.kT and softmax.v of a decode step); with few columns and many
        // k rows (softmax.v: 80 columns) the k rows are split over CTAs that leave f32 partial sums in act_scratch
        pl->kernel = PK_ROWVEC_MAT;
        pl->split = rowvec_mat_chunks((int)s.N, (int)s.K, (int)s.stacks, dev->sm_count);
        if (pl->split > 1) {
            pl->act_scratch_bytes = (uint64_t)s.stacks * (uint64_t)pl->split * (uint64_t)s.N * 4;
            cudaError_t e = cudaSetDevice(dev->ordinal);
            if (e == cudaSuccess) e = cudaMalloc(&pl->act_scratch, pl->act_scratch_bytes);
            if (e != cudaSuccess) {
                pl->act_scratch = nullptr;
                delete pl;
                return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                            std::string("plan scratch: ") + cudaGetErrorString(e));
            }
            pl->launches = 2;
        }
        pl->name = std::string("rowvec_mat_") + dtype_name(desc->rhs_dt) + (pl->split > 1 ? "_ksplit" + std::to_string(pl->split) : "");
    } else if (umma_eligible(*desc, s)) {
        pl->kernel = PK_GEMM_UMMA;
        pl->lhs_is_q = s.trans_out;
        const bool flatten = s.trans_out && s.lhs_stack == 1 && s.stacks > 1; // [B][N][M] with one shared W
        pl->R = (int)(s.trans_out ? (flatten ? s.stacks * s.N : s.N) : s.M);
        pl->S = (int)(s.trans_out ? s.M : s.N);
        pl->u_stacks = flatten ? 1 : (int)s.stacks;
        const int lhs_st = (int)s.lhs_stack, rhs_st = flatten ? 1 : (int)s.rhs_stack;
        pl->p_stack = s.trans_out ? rhs_st : lhs_st;
        pl->q_stack = s.trans_out ? lhs_st : rhs_st;
        pl->tf32x3 = desc->rhs_dt == RT_F32;
        pl->bn = pl->tf32x3 ? umma_tf32_pick_bn(pl->R, pl->S, pl->u_stacks, dev->sm_count)
                            : umma_pick_bn(pl->R, pl->S, pl->u_stacks, dev->sm_count);
        // problems that fill most of a wave of SM pairs with 256 x 256 tiles: two CTAs per tile (tcgen05 cta_group::2)
        if (!pl->tf32x3 && s.epilogue != RT_EPILOGUE_SILU_MUL && gemm_pair_enabled() && dev->sm_count >= 2 &&
            (long long)((pl->R + 255) / 256) * ((pl->S + 255) / 256) * pl->u_stacks >= gemm_pair_min_tiles(dev->sm_count))
            pl->bn = UMMA_BN_PAIR;
        pl->launches = 1;
        if (!s.trans_rhs) {
            pl->rhs_transpose = true;
            const uint64_t k_eff = pl->tf32x3 ? (uint64_t)s.K : (uint64_t)(s.K + 7) / 8 * 8;
            if (k_eff != (uint64_t)s.K) pl->k_pad = (int)k_eff;
            pl->act_scratch_bytes = (uint64_t)(s.rhs_stack * s.N) * k_eff * dtype_size(desc->rhs_dt);
            cudaError_t e = cudaSetDevice(dev->ordinal);
            if (e == cudaSuccess) e = cudaMalloc(&pl->act_scratch, pl->act_scratch_bytes);
            if (e == cudaSuccess && pl->k_pad) {
                pl->scratch_bytes = (uint64_t)(s.lhs_stack * s.M) * k_eff * 2;
                e = cudaMalloc(&pl->scratch, pl->scratch_bytes);
            }
            if (e != cudaSuccess) {
                if (pl->act_scratch) cudaFree(pl->act_scratch);
                pl->act_scratch = nullptr;
                pl->scratch = nullptr;
                delete pl;
                return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                            std::string("plan scratch: ") + cudaGetErrorString(e));
            }
            pl->launches += pl->k_pad ? 2 : 1;
        }
        if (pl->tf32x3 && umma_tf32_presplit_pays(pl->S, pl->bn)) {
            // P (the operand whose 128-row tiles every tile column reads) is split into hi and lo once
            // per launch, into this scratch, rather than by every CTA of its tile row.  A problem whose
            // P is too large for that keeps the split inside the GEMM.
            const uint64_t bytes = (uint64_t)pl->p_stack * (uint64_t)pl->R * (uint64_t)s.K * 8;
            if (bytes <= (1ull << 30)) {
                cudaError_t e = cudaSetDevice(dev->ordinal);
                if (e == cudaSuccess) e = cudaMalloc(&pl->scratch, bytes);
                if (e != cudaSuccess) {
                    pl->scratch = nullptr;
                    delete pl;
                    return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                                std::string("plan scratch: ") + cudaGetErrorString(e));
                }
                pl->scratch_bytes = bytes;
                pl->launches++;
            }
        }
        if (is_quantized(desc->lhs_dt) && pl->tf32x3) {
            pl->wdq_bytes = (uint64_t)(s.lhs_stack * s.M * s.K) * 4;
            cudaError_t e = cudaSetDevice(dev->ordinal);
            if (e == cudaSuccess) e = cudaMalloc(&pl->wdq, pl->wdq_bytes);
            if (e != cudaSuccess) {
                pl->wdq = nullptr;
                delete pl;
                return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA, std::string("plan scratch: ") + cudaGetErrorString(e));
            }
            pl->launches++;
        } else if (is_quantized(desc->lhs_dt)) {
            pl->scratch_bytes = (uint64_t)(s.lhs_stack * s.M * s.K) * 2;
            cudaError_t e = cudaSetDevice(dev->ordinal);
            if (e == cudaSuccess) e = cudaMalloc(&pl->scratch, pl->scratch_bytes);
            if (e != cudaSuccess) {
                pl->scratch = nullptr;
                delete pl;
                return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                            std::string("plan scratch: ") + cudaGetErrorString(e));
            }
            pl->launches = 2;
            // tcgen05.mma kind::f16 takes one 16-bit format for both operands: the dequantised weights
            // are f16 (bf16 would drop 3 of their 11 significant bits), so bf16 activations are cast, each row
            // with a power-of-two factor that brings it into f16's range and that the epilogue puts back
            if (desc->rhs_dt == RT_BF16) {
                pl->act_scale_off = ((uint64_t)(s.rhs_stack * s.N * s.K) * 2 + 255) / 256 * 256;
                pl->act_scratch_bytes = pl->act_scale_off + (uint64_t)(s.rhs_stack * s.N) * 4;
                e = cudaMalloc(&pl->act_scratch, pl->act_scratch_bytes);
                if (e != cudaSuccess) {
                    pl->act_scratch = nullptr;
                    delete pl;
                    return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                                std::string("plan scratch: ") + cudaGetErrorString(e));
                }
                pl->launches = 3;
            }
        }
        pl->name = std::string(pl->tf32x3 ? "gemm_umma_tf32x3_" : "gemm_umma_") + dtype_name(desc->lhs_dt) + "_" + dtype_name(desc->rhs_dt) +
                   (pl->bn == UMMA_BN_PAIR ? std::string("_pair256x256") : "_bn" + std::to_string(pl->bn)) + (pl->scratch && !pl->k_pad ? (pl->tf32x3 ? "_presplit" : "_dequant_prepass") : "") + (pl->wdq ? "_dequant_prepass" : "") +
                   (pl->rhs_transpose ? "_rhs_transposed" : "") + (pl->k_pad ? "_kpad" + std::to_string(pl->k_pad) : "");
    } else if (s.N == 1 && !s.trans_lhs) {
        pl->kernel = PK_GEMV_SIMT;
        pl->name = std::string("gemv_simt_") + dtype_name(desc->lhs_dt) + "_" + dtype_name(desc->rhs_dt);
    } else {
        pl->kernel = PK_GEMM_SIMT;
        pl->name = std::string("gemm_simt_") + dtype_name(desc->lhs_dt) + "_" + dtype_name(desc->rhs_dt);
    }
    if (s.epilogue == RT_EPILOGUE_SILU_MUL) {
        if (pl->kernel == PK_GEMM_UMMA && !pl->tf32x3) {
            pl->name += "_silu_mul_paired_tiles"; // gate and up rows of a column meet in one tile
        } else {
            pl->pair = true;
            pl->chain_ok = false;
            p.epilogue = RT_EPILOGUE_NONE;
            pl->pair_bytes = (uint64_t)(s.stacks * s.N * s.M) * dtype_size(s.out_dt);
            if (pl->pair_bytes) {
                cudaError_t e = cudaSetDevice(dev->ordinal);
                if (e == cudaSuccess) e = cudaMalloc(&pl->pair_scratch, pl->pair_bytes);
                if (e != cudaSuccess) {
                    pl->pair_scratch = nullptr;
                    delete pl;
                    return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA,
                                std::string("plan scratch: ") + cudaGetErrorString(e));
                }
            }
            pl->launches++;
            pl->name += "+silu_mul";
        }
    }
    if (empty) pl->launches = 0;
    *plan = pl;
    return RT_OK;
}

// Gives the caller's hold on the plan back; the device's cache keeps its own until rt_device_destroy.
rt_status rt_plan_destroy(rt_plan *plan) {
    if (!plan) return RT_OK;
    rt_device *dev = plan->dev;
    std::lock_guard<std::mutex> lk(dev->plan_mu);
    if (--plan->refs <= 0) {
        dev->plans.erase(plan->key);
        delete plan;
    }
    return RT_OK;
}

rt_status rt_plan_forget_weights(rt_plan *plan) {
    if (!plan) return fail(RT_ERR_ARG, "rt_plan_forget_weights: null plan");
    CUDA_TRY(cudaSetDevice(plan->dev->ordinal));
    std::lock_guard<std::mutex> lk(plan->weights_mu);
    for (auto &kv : plan->kept_weights) cudaFree(kv.second);
    plan->kept_weights.clear();
    return RT_OK;
}

// sizeof / offsetof of the public structs, for bindings to check their mirrors against: the entries are
// {sizeof(rt_shape), offsetof dims, sizeof(rt_segment), sizeof(rt_matmul_desc), offsetof lhs_shape, rhs_shape, bias_shape,
//  has_bias, epilogue, sizeof(rt_gemm_spec), offsetof out_dt, lhs_stack, dim_inner, is_gemv, sizeof(rt_launch_opts), offsetof
//  outs, out_ld, out_col, sizeof(rt_dispatch), offsetof opts, sizeof(rt_gguf_value), offsetof str,
//  sizeof(rt_gguf_tensor_info), offsetof shape, nbytes, sizeof(rt_usage_record), offsetof producer, sizeof(rt_node_tensors),
//  sizeof(rt_mlp_desc), offsetof fc2, w1, out}
int32_t rt_abi_layout(uint64_t *out, int32_t n) {
    const uint64_t v[] = {
        sizeof(rt_shape), offsetof(rt_shape, dims), sizeof(rt_segment),
        sizeof(rt_matmul_desc), offsetof(rt_matmul_desc, lhs_shape), offsetof(rt_matmul_desc, rhs_shape), offsetof(rt_matmul_desc, bias_shape),
        offsetof(rt_matmul_desc, has_bias), offsetof(rt_matmul_desc, epilogue),
        sizeof(rt_gemm_spec), offsetof(rt_gemm_spec, out_dt), offsetof(rt_gemm_spec, lhs_stack), offsetof(rt_gemm_spec, dim_inner), offsetof(rt_gemm_spec, is_gemv),
        sizeof(rt_launch_opts), offsetof(rt_launch_opts, outs), offsetof(rt_launch_opts, out_ld), offsetof(rt_launch_opts, out_col),
        sizeof(rt_dispatch), offsetof(rt_dispatch, opts),
        sizeof(rt_gguf_value), offsetof(rt_gguf_value, str),
        sizeof(rt_gguf_tensor_info), offsetof(rt_gguf_tensor_info, shape), offsetof(rt_gguf_tensor_info, nbytes),
        sizeof(rt_usage_record), offsetof(rt_usage_record, producer), sizeof(rt_node_tensors),
        sizeof(rt_mlp_desc), offsetof(rt_mlp_desc, fc2), offsetof(rt_mlp_desc, w1), offsetof(rt_mlp_desc, out)};
    const int32_t count = (int32_t)(sizeof(v) / sizeof(v[0]));
    for (int32_t i = 0; i < count && i < n; i++) out[i] = v[i];
    return count;
}

rt_status rt_plan_spec(const rt_plan *plan, rt_gemm_spec *spec) {
    if (!plan || !spec) return fail(RT_ERR_ARG, "rt_plan_spec: null argument");
    fill_public_spec(plan->spec, spec);
    return RT_OK;
}

const char *rt_plan_kernel(const rt_plan *plan) { return plan ? plan->name.c_str() : ""; }
int32_t rt_plan_launches(const rt_plan *plan) { return plan ? plan->launches : 0; }

static MatmulParams bound_params(const rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out) {
    MatmulParams p = plan->params;
    p.lhs = lhs;
    p.lhs_scales = plan->lhs_scale_offset ? (const void *)((const char *)lhs + plan->lhs_scale_offset) : nullptr;
    p.rhs = rhs;
    p.bias = plan->spec.has_bias ? bias : nullptr;
    p.out = out;
    return p;
}

rt_status rt_matmul_launch(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream) {
    return rt_matmul_launch_ex(plan, lhs, rhs, bias, out, stream, nullptr);
}

rt_status rt_matmul_launch_ex(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream,
                              const rt_launch_opts *opts) {
    return launch_node(plan, lhs, rhs, bias, out, stream, opts, nullptr);
}

} // extern "C"

// One node's launches.  `ov` names scratch areas that take the place of the plan's own (an executable's arena).
static rt_status launch_node(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream,
                             const rt_launch_opts *opts, const ScratchSet *ov) {
    if (!plan) return fail(RT_ERR_ARG, "rt_matmul_launch: null plan");
    const uint32_t flags = opts ? opts->flags : 0;
    const bool scatter = opts && opts->n_out > 0;
    if (scatter) {
        if (plan->kernel != PK_GEMM_UMMA) return fail(RT_ERR_UNSUPPORTED, "scattered outputs are only taken by the tensor-core GEMM");
        if (opts->n_out > RT_MAX_PEERS || opts->out_col < 0 || opts->out_ld < opts->out_col + plan->S)
            return fail(RT_ERR_ARG, "rt_matmul_launch_ex: bad scatter description");
        for (int d = 0; d < opts->n_out; d++)
            if (!opts->outs[d]) return fail(RT_ERR_ARG, "rt_matmul_launch_ex: null scatter destination");
    }
    const Spec &s = plan->spec;
    if (scatter && s.epilogue == RT_EPILOGUE_SILU_MUL)
        return fail(RT_ERR_UNSUPPORTED, "scattered outputs are not taken with RT_EPILOGUE_SILU_MUL");
    if (plan->launches == 0) return RT_OK; // empty output
    void *const scratch = ov && ov->scratch ? ov->scratch : plan->scratch;
    void *const act_scratch = ov && ov->act ? ov->act : plan->act_scratch;
    void *const pair_scratch = ov && ov->pair ? ov->pair : plan->pair_scratch;
    void *const user_out = out;
    if (plan->pair) out = pair_scratch; // the plain node's [.., 2*ff] result; folded after the switch
    if (!lhs || !rhs || (!user_out && !(opts && opts->n_out > 0)) || (s.has_bias && !bias))
        return fail(RT_ERR_ARG, "rt_matmul_launch: null operand");
    if (user_out == lhs || user_out == rhs || (s.has_bias && user_out == bias))
        return fail(RT_ERR_INVARIANT, "Matmul is never in place: out aliases an operand");
    CUDA_TRY(cudaSetDevice(plan->dev->ordinal));
    cudaStream_t st = stream ? (cudaStream_t)stream : plan->dev->stream;
    MatmulParams p = bound_params(plan, lhs, rhs, bias, out);
    cudaError_t e = cudaSuccess;
    switch (plan->kernel) {
    case PK_Q8_GEMV_MMA:
        // the kernel fetches weight rows with bulk copies and activations with 16-byte loads
        if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) % 16 != 0)
            return fail(RT_ERR_ARG, "rt_matmul_launch: lhs and rhs must be 16-byte aligned");
        e = launch_q8_gemv_mma(p, s.desc.lhs_dt == RT_Q8_0F, plan->nv, plan->split, (flags & RT_LAUNCH_LHS_CONSTANT) != 0, st);
        for (int done = plan->nv; e == cudaSuccess && done < plan->nv + plan->nv2; done += 16) {
            MatmulParams p2 = p; // vectors done.. : rhs rows and (trans_out) output rows of the same problem
            p2.rhs = (const char *)rhs + (size_t)done * (size_t)s.K * 2;
            p2.out = (char *)out + (size_t)done * (size_t)s.M * 2;
            const int nv = std::min(16, plan->nv + plan->nv2 - done);
            e = launch_q8_gemv_mma(p2, s.desc.lhs_dt == RT_Q8_0F, nv, plan->split, (flags & RT_LAUNCH_LHS_CONSTANT) != 0, st);
        }
        break;
    case PK_Q4K_GEMV:
        if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) % 16 != 0)
            return fail(RT_ERR_ARG, "rt_matmul_launch: lhs and rhs must be 16-byte aligned");
        e = launch_q4k_gemv(p, plan->nv, plan->split, (flags & RT_LAUNCH_LHS_CONSTANT) != 0, st);
        break;
    case PK_Q4K_GEMV_UMMA:
        if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) % 16 != 0)
            return fail(RT_ERR_ARG, "rt_matmul_launch: lhs and rhs must be 16-byte aligned");
        e = launch_q4k_gemv_umma(p, plan->nv, plan->q4k_umma, (flags & RT_LAUNCH_LHS_CONSTANT) != 0, st);
        break;
    case PK_Q8_GEMV_UMMA:
        if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) % 16 != 0)
            return fail(RT_ERR_ARG, "rt_matmul_launch: lhs and rhs must be 16-byte aligned");
        e = launch_q8_gemv_umma(p, plan->gemv_umma, (flags & RT_LAUNCH_LHS_CONSTANT) != 0, st);
        break;
    case PK_GEMV_SIMT:
        e = launch_matmul_simt(p, s.desc.lhs_dt, s.desc.rhs_dt, true, st);
        break;
    case PK_ROWVEC_MAT:
        e = launch_rowvec_mat(p, s.desc.rhs_dt, plan->split, static_cast<float *>(act_scratch), st);
        break;
    case PK_GEMM_SIMT:
        e = launch_matmul_simt(p, s.desc.lhs_dt, s.desc.rhs_dt, false, st);
        break;
    case PK_GEMM_UMMA: {
        // tensor maps want 16-byte aligned bases, and the pre-passes (dequantise, cast, pad) read 16 bytes per load
        if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) % 16 != 0)
            return fail(RT_ERR_ARG, "rt_matmul_launch: lhs and rhs must be 16-byte aligned");
        if (plan->tf32x3) {
            if (scatter) return fail(RT_ERR_UNSUPPORTED, "scattered outputs are not taken by the f32 GEMM");
            const void *r32 = rhs;
            if (plan->rhs_transpose) {
                e = launch_transpose(rhs, act_scratch, (int)s.rhs_stack, (int)s.K, (int)s.N, (int)s.K, 4, st);
                if (e != cudaSuccess) break;
                r32 = act_scratch;
            }
            const void *wl = lhs;
            if (plan->wdq_bytes) {
                // Q8_0F weights as f32; a weight flagged constant keeps its copy with the plan, as the 16-bit route does
                void *dst = ov && ov->wdq ? ov->wdq : plan->wdq;
                bool have = false;
                if (flags & RT_LAUNCH_LHS_CONSTANT) {
                    void *kept = kept_weight_copy(plan, lhs, st, &have, plan->wdq_bytes);
                    if (kept) dst = kept;
                }
                if (!have) {
                    e = launch_dequant(s.desc.lhs_dt, (long long)(s.lhs_stack * s.M * s.K), lhs, p.lhs_scales, dst, RT_F32,
                                       plan->dev->sm_count, st);
                    if (e != cudaSuccess) break;
                }
                wl = dst;
            }
            const void *P = plan->lhs_is_q ? r32 : wl, *Q = plan->lhs_is_q ? wl : r32;
            e = launch_gemm_umma_tf32x3(P, Q, out, plan->R, plan->S, (int)s.K, plan->u_stacks, plan->p_stack, plan->q_stack, p.bias,
                                        p.bias_dt, s.has_bias ? BIAS_PER_N : BIAS_NONE, p.epilogue, plan->bn, plan->scratch ? scratch : nullptr,
                                        plan->dev->sm_count, st);
            break;
        }
        const void *w = lhs;
        rt_dtype w_dt = s.desc.lhs_dt;
        const int k_eff = plan->k_pad ? plan->k_pad : (int)s.K;
        if (plan->k_pad) {
            e = launch_pad_rows16(lhs, scratch, (long long)(s.lhs_stack * s.M), (int)s.K, plan->k_pad, plan->dev->sm_count, st);
            if (e != cudaSuccess) break;
            w = scratch;
        } else if (plan->scratch) {
            // A weight flagged constant is dequantised once and its f16 copy kept with the plan (the first launch with a
            // new weight allocates: make it outside any stream capture); any other lhs goes through the plan's own scratch
            // on every launch.
            void *dst = scratch;
            bool have = false;
            if (flags & RT_LAUNCH_LHS_CONSTANT) {
                void *kept = kept_weight_copy(plan, lhs, st, &have, plan->scratch_bytes);
                if (kept) dst = kept;
            }
            if (!have) {
                e = launch_dequant(s.desc.lhs_dt, (long long)(s.lhs_stack * s.M * s.K), lhs, p.lhs_scales, dst, RT_F16,
                                   plan->dev->sm_count, st);
                if (e != cudaSuccess) break;
            }
            w = dst;
            w_dt = RT_F16;
        }
        const void *x = rhs;
        rt_dtype x_dt = s.desc.rhs_dt;
        float *x_scale = nullptr;
        if (plan->rhs_transpose) {
            e = launch_transpose(rhs, act_scratch, (int)s.rhs_stack, (int)s.K, (int)s.N, k_eff, 2, st);
            if (e != cudaSuccess) break;
            x = act_scratch;
        } else if (plan->act_scratch) {
            x_scale = reinterpret_cast<float *>(static_cast<char *>(act_scratch) + plan->act_scale_off);
            e = launch_cast_bf16_f16_rows(rhs, act_scratch, x_scale, (long long)(s.rhs_stack * s.N), (int)s.K, plan->dev->sm_count, st);
            if (e != cudaSuccess) break;
            x = act_scratch;
            x_dt = RT_F16;
        }
        const void *P = plan->lhs_is_q ? x : w, *Q = plan->lhs_is_q ? w : x;
        const rt_dtype p_dt = plan->lhs_is_q ? x_dt : w_dt, q_dt = plan->lhs_is_q ? w_dt : x_dt;
        UmmaScatter sc{};
        if (scatter) {
            if (!plan->lhs_is_q || plan->u_stacks != 1)
                return fail(RT_ERR_UNSUPPORTED, "scattered outputs need trans_out and one shared weight");
            sc.n_out = opts->n_out;
            for (int d = 0; d < opts->n_out; d++) sc.outs[d] = opts->outs[d];
            sc.out_ld = opts->out_ld;
            sc.out_col = opts->out_col;
        }
        e = launch_gemm_umma(P, p_dt, Q, q_dt, out, s.out_dt, plan->R, plan->S, k_eff, plan->u_stacks, plan->p_stack,
                             plan->q_stack, p.bias, p.bias_dt, s.has_bias ? BIAS_PER_N : BIAS_NONE, p.epilogue, plan->bn,
                             plan->dev->sm_count, st, scatter ? &sc : nullptr, plan->lhs_is_q ? x_scale : nullptr,
                             plan->lhs_is_q ? nullptr : x_scale);
        break;
    }
    }
    if (e == cudaSuccess && plan->pair)
        e = launch_silu_mul(pair_scratch, user_out, (long long)(s.stacks * s.N), (int)(s.M / 2), s.out_dt, plan->dev->sm_count, st);
    if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("kernel launch (") + plan->name + "): " + cudaGetErrorString(e));
    return RT_OK;
}

extern "C" {


static rt_status dispatch_nodes(rt_executable *exe, cudaStream_t st) {
    for (size_t i = 0; i < exe->nodes.size(); i++) {
        const rt_dispatch &n = exe->nodes[i];
        rt_status s = launch_node(n.plan, n.lhs, n.rhs, n.bias, n.out, (void *)st, &n.opts, &exe->scratch[i]);
        if (s != RT_OK) return s;
    }
    return RT_OK;
}

rt_status rt_executable_create(rt_device *dev, const rt_dispatch *nodes, int32_t n_nodes, int32_t use_graph, rt_executable **exe) {
    return rt_executable_create_planned(dev, nodes, nullptr, n_nodes, nullptr, 0, use_graph, exe);
}

rt_status rt_executable_create_planned(rt_device *dev, const rt_dispatch *nodes, const rt_node_tensors *ids, int32_t n_nodes,
                                       const uint64_t *tensor_bytes, int32_t n_tensors, int32_t use_graph, rt_executable **exe) {
    if (!dev || !exe || (n_nodes > 0 && !nodes) || n_nodes < 0 || n_tensors < 0 || (n_tensors > 0 && (!tensor_bytes || !ids)))
        return fail(RT_ERR_ARG, "rt_executable_create: bad argument");
    std::unique_ptr<rt_executable> x(new (std::nothrow) rt_executable());
    if (!x) return fail(RT_ERR_NOMEM, "out of host memory");
    x->dev = dev;
    for (int i = 0; i < n_nodes; i++) {
        if (!nodes[i].plan || nodes[i].plan->dev != dev)
            return fail(RT_ERR_ARG, "rt_executable_create: node without a plan of this device");
        x->nodes.push_back(nodes[i]);
        x->launches += nodes[i].plan->launches;
    }
    x->scratch.resize((size_t)n_nodes);
    x->tensors.assign((size_t)n_tensors, nullptr);

    // usage records (allocator.rs:168-207): intermediates first, then each node's scratch areas
    std::vector<int> producer((size_t)n_tensors, -1), last((size_t)n_tensors, -1);
    for (int i = 0; ids && i < n_nodes; i++) {
        const rt_node_tensors &t = ids[i];
        const int reads[3] = {t.lhs, t.rhs, x->nodes[(size_t)i].plan->spec.has_bias ? t.bias : -1};
        for (int id : reads) {
            if (id < 0) continue;
            if (id >= n_tensors) return fail(RT_ERR_ARG, "rt_executable_create: intermediate id out of range");
            if (producer[(size_t)id] < 0 || producer[(size_t)id] >= i)
                return fail(RT_ERR_ARG, "rt_executable_create: node " + std::to_string(i) + " reads intermediate " +
                                            std::to_string(id) + " before a node produced it");
            last[(size_t)id] = i;
        }
        if (t.lhs >= 0 && (x->nodes[(size_t)i].opts.flags & RT_LAUNCH_LHS_CONSTANT))
            return fail(RT_ERR_ARG, "rt_executable_create: an intermediate cannot be flagged RT_LAUNCH_LHS_CONSTANT");
        if (t.out >= 0) {
            if (t.out >= n_tensors) return fail(RT_ERR_ARG, "rt_executable_create: intermediate id out of range");
            if (x->nodes[(size_t)i].opts.n_out > 0)
                return fail(RT_ERR_ARG, "rt_executable_create: a scattered output cannot be an intermediate");
            const Spec &sp = x->nodes[(size_t)i].plan->spec;
            rt_segment seg[2];
            int nseg = 0;
            uint64_t need = 0;
            Status st = dtype_segments(sp.out_dt, (uint64_t)numel(sp.out_shape), seg, &nseg);
            if (!st.ok()) return fail(st);
            for (int k = 0; k < nseg; k++) need += seg[k].size;
            if (tensor_bytes[t.out] < need)
                return fail(RT_ERR_ARG, "rt_executable_create: intermediate " + std::to_string(t.out) + " is smaller than node " +
                                            std::to_string(i) + "'s output");
            if (producer[(size_t)t.out] < 0) producer[(size_t)t.out] = i;
            last[(size_t)t.out] = i;
        }
    }
    // Weights flagged constant get their dequantised copy now (outside the capture below), filled on the device's
    // stream and complete when this call returns; such a node then needs no dequantising scratch.
    bool filled_any = false;
    std::vector<bool> kept((size_t)n_nodes, false);
    CUDA_TRY(cudaSetDevice(dev->ordinal));
    for (int i = 0; i < n_nodes; i++) {
        const rt_dispatch &n = x->nodes[(size_t)i];
        rt_plan *pl = n.plan;
        const bool f32_route = pl->kernel == PK_GEMM_UMMA && pl->tf32x3 && pl->wdq_bytes;
        const bool f16_route = pl->kernel == PK_GEMM_UMMA && !pl->tf32x3 && !pl->k_pad && pl->scratch;
        if (!(n.opts.flags & RT_LAUNCH_LHS_CONSTANT) || !(f32_route || f16_route) || !n.lhs || pl->launches == 0) continue;
        bool filled = false;
        void *copy = kept_weight_copy(pl, n.lhs, dev->stream, &filled, f32_route ? pl->wdq_bytes : pl->scratch_bytes);
        if (!copy) continue;
        if (!filled) {
            const Spec &sp = pl->spec;
            const void *scales = pl->lhs_scale_offset ? (const void *)((const char *)n.lhs + pl->lhs_scale_offset) : nullptr;
            cudaError_t e = launch_dequant(sp.desc.lhs_dt, (long long)(sp.lhs_stack * sp.M * sp.K), n.lhs, scales, copy,
                                           f32_route ? RT_F32 : RT_F16, dev->sm_count, dev->stream);
            if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("dequantise (") + pl->name + "): " + cudaGetErrorString(e));
            filled_any = true;
        }
        kept[(size_t)i] = true;
        x->launches -= 1; // this node's dispatches go without the dequantising pass
    }
    if (filled_any) CUDA_TRY(cudaStreamSynchronize(dev->stream));

    std::vector<rt_usage_record> rec;
    std::vector<void **> slot; // where each record's address goes
    for (int k = 0; k < n_tensors; k++) {
        if (producer[(size_t)k] < 0) continue; // never produced: never bound
        rec.push_back({tensor_bytes[k], producer[(size_t)k], last[(size_t)k]});
        slot.push_back(&x->tensors[(size_t)k]);
    }
    for (int i = 0; i < n_nodes; i++) {
        const rt_plan *pl = x->nodes[(size_t)i].plan;
        if (pl->launches == 0) continue;
        ScratchSet &sc = x->scratch[(size_t)i];
        // (the f32 route's `scratch` is the activations' hi / lo split, needed at every dispatch; its kept copy is `wdq`)
        if (pl->scratch_bytes && !(kept[(size_t)i] && !pl->tf32x3)) { rec.push_back({pl->scratch_bytes, i, i}); slot.push_back(&sc.scratch); }
        if (pl->wdq_bytes && !kept[(size_t)i]) { rec.push_back({pl->wdq_bytes, i, i}); slot.push_back(&sc.wdq); }
        if (pl->act_scratch_bytes) { rec.push_back({pl->act_scratch_bytes, i, i}); slot.push_back(&sc.act); }
        if (pl->pair_bytes) { rec.push_back({pl->pair_bytes, i, i}); slot.push_back(&sc.pair); }
    }
    ArenaPlan ap;
    Status pst = plan_arena(rec.data(), (int32_t)rec.size(), 256, &ap);
    if (!pst.ok()) return fail(pst);
    x->arena_bytes = ap.arena_bytes;
    x->n_objects = (int)ap.object_bytes.size();
    for (const rt_usage_record &r : rec) x->record_bytes += r.size;
    if (ap.arena_bytes) {
        cudaError_t e = cudaMalloc(&x->arena, ap.arena_bytes);
        if (e != cudaSuccess) {
            x->arena = nullptr;
            return fail(e == cudaErrorMemoryAllocation ? RT_ERR_NOMEM : RT_ERR_CUDA, std::string("executable arena: ") + cudaGetErrorString(e));
        }
    }
    for (size_t r = 0; r < rec.size(); r++) *slot[r] = (char *)x->arena + ap.offset[r];
    for (int i = 0; ids && i < n_nodes; i++) {
        rt_dispatch &n = x->nodes[(size_t)i];
        if (ids[i].lhs >= 0) n.lhs = x->tensors[(size_t)ids[i].lhs];
        if (ids[i].rhs >= 0) n.rhs = x->tensors[(size_t)ids[i].rhs];
        if (ids[i].bias >= 0 && n.plan->spec.has_bias) n.bias = x->tensors[(size_t)ids[i].bias];
        if (ids[i].out >= 0) n.out = x->tensors[(size_t)ids[i].out];
    }
    for (const rt_dispatch &n : x->nodes)
        if (n.out && (n.out == n.lhs || n.out == n.rhs || (n.plan->spec.has_bias && n.out == n.bias)))
            return fail(RT_ERR_INVARIANT, "Matmul is never in place: out aliases an operand");

    // A list of tensor-memory Q8_0 GEMVs over constant weights runs as one persistent kernel.
    if (use_graph && n_nodes >= 2 && chain_enabled()) {
        bool all = true;
        std::vector<MatmulParams> ps;
        for (const rt_dispatch &n : x->nodes) {
            if (!n.plan->chain_ok || !(n.opts.flags & RT_LAUNCH_LHS_CONSTANT) || n.opts.n_out > 0 || !n.lhs || !n.rhs ||
                !n.out || (n.plan->spec.has_bias && !n.bias)) {
                all = false;
                break;
            }
            ps.push_back(bound_params(n.plan, n.lhs, n.rhs, n.bias, n.out));
        }
        if (all) {
            std::string why;
            cudaError_t e = gemv_chain_create(ps, dev->ordinal, dev->sm_count, &x->chain, &why);
            if (e != cudaSuccess) return fail(RT_ERR_CUDA, std::string("gemv_chain_create: ") + cudaGetErrorString(e));
            if (x->chain) {
                x->how = gemv_chain_name(x->chain);
                x->launches = 1;
                *exe = x.release();
                return RT_OK;
            }
        }
    }
    if (use_graph && x->launches > 0) {
        x->how = "graph";
        cudaError_t e = cudaSuccess;
        cudaStream_t cap = nullptr;
        e = cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamBeginCapture(cap, cudaStreamCaptureModeRelaxed);
        rt_status rs = RT_OK;
        if (e == cudaSuccess) {
            rs = dispatch_nodes(x.get(), cap);
            cudaError_t e2 = cudaStreamEndCapture(cap, &x->graph);
            if (rs == RT_OK) e = e2;
        }
        if (rs == RT_OK && e == cudaSuccess) e = cudaGraphInstantiate(&x->exec, x->graph, 0);
        if (cap) cudaStreamDestroy(cap);
        if (rs != RT_OK || e != cudaSuccess) {
            std::string msg = rs != RT_OK ? last_error() : std::string("graph capture: ") + cudaGetErrorString(e);
            return fail(rs != RT_OK ? rs : RT_ERR_CUDA, msg);
        }
    }
    *exe = x.release();
    return RT_OK;
}

rt_status rt_executable_arena(const rt_executable *exe, uint64_t *arena_bytes, int32_t *n_objects, uint64_t *record_bytes) {
    if (!exe) return fail(RT_ERR_ARG, "rt_executable_arena: null executable");
    if (arena_bytes) *arena_bytes = exe->arena_bytes;
    if (n_objects) *n_objects = exe->n_objects;
    if (record_bytes) *record_bytes = exe->record_bytes;
    return RT_OK;
}

void *rt_executable_tensor(const rt_executable *exe, int32_t id) {
    if (!exe || id < 0 || (size_t)id >= exe->tensors.size()) return nullptr;
    return exe->tensors[(size_t)id];
}

rt_status rt_mlp_create(rt_device *dev, const rt_mlp_desc *mlp, int32_t use_graph, rt_executable **exe) {
    if (!dev || !mlp || !exe) return fail(RT_ERR_ARG, "rt_mlp_create: null argument");
    for (const rt_matmul_desc *d : {&mlp->fc1, &mlp->fc2})
        if (!(d->trans_rhs && d->trans_out && !d->trans_lhs))
            return fail(RT_ERR_INVARIANT, "rt_mlp_create: fc1 and fc2 are Linear nodes (trans_rhs, trans_out)");
    if (mlp->fc2.epilogue != RT_EPILOGUE_NONE) return fail(RT_ERR_ARG, "rt_mlp_create: fc2 carries no activation");
    rt_plan *p1 = nullptr, *p2 = nullptr;
    rt_status rs = rt_matmul_plan(dev, &mlp->fc1, &p1);
    if (rs != RT_OK) return rs;
    rs = rt_matmul_plan(dev, &mlp->fc2, &p2);
    if (rs != RT_OK) {
        rt_plan_destroy(p1);
        return rs;
    }
    auto give_back = [&]() { rt_plan_destroy(p1); rt_plan_destroy(p2); };
    // the hidden tensor is fc1's output and fc2's rhs
    const Dims hid = p1->spec.out_shape, rhs2 = to_dims(mlp->fc2.rhs_shape);
    if (hid != rhs2 || p1->spec.out_dt != mlp->fc2.rhs_dt) {
        give_back();
        return fail(RT_ERR_SHAPE, "rt_mlp_create: fc1 produces " + dims_str(hid) + " " + dtype_name(p1->spec.out_dt) + ", fc2 takes " +
                                      dims_str(rhs2) + " " + dtype_name(mlp->fc2.rhs_dt));
    }
    rt_segment seg[2];
    int nseg = 0;
    uint64_t hidden_bytes = 0;
    Status st = dtype_segments(p1->spec.out_dt, (uint64_t)numel(hid), seg, &nseg);
    if (!st.ok()) {
        give_back();
        return fail(st);
    }
    for (int k = 0; k < nseg; k++) hidden_bytes += seg[k].size;
    rt_dispatch nodes[2] = {};
    nodes[0].plan = p1; nodes[0].lhs = mlp->w1; nodes[0].rhs = mlp->x; nodes[0].bias = mlp->b1;
    nodes[0].opts.flags = RT_LAUNCH_LHS_CONSTANT;
    nodes[1].plan = p2; nodes[1].lhs = mlp->w2; nodes[1].bias = mlp->b2; nodes[1].out = mlp->out;
    nodes[1].opts.flags = RT_LAUNCH_LHS_CONSTANT;
    const rt_node_tensors ids[2] = {{-1, -1, -1, 0}, {-1, 0, -1, -1}};
    rs = rt_executable_create_planned(dev, nodes, ids, 2, &hidden_bytes, 1, use_graph, exe);
    // The executable does not own plans; the device's cache keeps both alive until rt_device_destroy, so the
    // holds taken here can go back at once.
    give_back();
    return rs;
}

rt_status rt_executable_dispatch(rt_executable *exe, void *stream) {
    if (!exe) return fail(RT_ERR_ARG, "rt_executable_dispatch: null executable");
    cudaStream_t st = stream ? (cudaStream_t)stream : exe->dev->stream;
    if (exe->chain && !exe->chain_refused) {
        CUDA_TRY(cudaSetDevice(exe->dev->ordinal));
        cudaError_t e = gemv_chain_launch(exe->chain, st);
        if (e == cudaSuccess) return RT_OK;
        // a refused launch (e.g. the cooperative grid does not fit beside other work) is not sticky
        cudaGetLastError();
        exe->chain_refused = true;
        exe->how = std::string("nodes (chain launch refused: ") + cudaGetErrorString(e) + ")";
        exe->launches = 0;
        for (auto &n : exe->nodes) exe->launches += n.plan->launches;
    }
    if (exe->exec) {
        CUDA_TRY(cudaSetDevice(exe->dev->ordinal));
        CUDA_TRY(cudaGraphLaunch(exe->exec, st));
        return RT_OK;
    }
    return dispatch_nodes(exe, st);
}

rt_status rt_executable_destroy(rt_executable *exe) {
    if (!exe) return RT_OK;
    delete exe;
    return RT_OK;
}

int32_t rt_executable_launches(const rt_executable *exe) { return exe ? exe->launches : 0; }
const char *rt_executable_kernel(const rt_executable *exe) { return exe ? exe->how.c_str() : ""; }

rt_status rt_dequantize_device(rt_device *dev, rt_dtype dt, uint64_t numel, const void *src, void *dst, void *stream) {
    if (!dev || !src || !dst) return fail(RT_ERR_ARG, "rt_dequantize_device: null argument");
    if (!dtype_valid(dt) || !is_quantized(dt)) return fail(RT_ERR_DTYPE, "rt_dequantize_device: not a block format");
    rt_segment seg[2];
    int n = 0;
    Status st = dtype_segments(dt, numel, seg, &n);
    if (!st.ok()) return fail(st);
    CUDA_TRY(cudaSetDevice(dev->ordinal));
    const void *scales = n == 2 ? (const void *)((const char *)src + seg[1].offset) : nullptr;
    cudaStream_t s = stream ? (cudaStream_t)stream : dev->stream;
    CUDA_TRY(launch_dequant(dt, (long long)numel, src, scales, dst, dt == RT_Q8_0H ? RT_F16 : RT_F32, dev->sm_count, s));
    return RT_OK;
}

} // extern "C"
