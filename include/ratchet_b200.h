/*
 * ratchet_b200 — C ABI of the B200 (sm_100a) implementation of ratchet-core's Matmul path.
 *
 * The reference (FL33TW00D/ratchet) is Rust + WebGPU and has no FFI of its own; each entry
 * point below names the Rust item whose role it takes, so that a `-sys` crate can bind these
 * symbols and ratchet-core's `Tensor::gemm -> LazyOp::Matmul -> compile -> dispatch` path
 * can call them instead of building WGSL.  Paths are relative to the reference project.
 *
 * Conventions
 *  - every function returns an rt_status; on failure `rt_last_error()` gives a thread-local
 *    message.  Where the reference panics (invariant violations) this library returns
 *    RT_ERR_INVARIANT / RT_ERR_DTYPE instead of aborting; where it returns an error
 *    (`anyhow::bail!`) this library returns RT_ERR_SHAPE.
 *  - shapes are row-major, at most RT_MAX_RANK dimensions, int64 extents.
 *  - device pointers are plain `void*` obtained from rt_buffer_ptr() or from any other
 *    CUDA allocator in the same process (cudaMalloc, a framework's caching allocator).
 *  - nothing on the launch path allocates, synchronises the device, or falls back to the CPU.
 */
#ifndef RATCHET_B200_H
#define RATCHET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RT_MAX_RANK 8
#define RT_MAX_PEERS 8

typedef enum rt_status {
    RT_OK = 0,
    RT_ERR_SHAPE = 1,       /* reference: anyhow error from Matmul::compute_c_shape (ops/matmul.rs:284-361) */
    RT_ERR_DTYPE = 2,       /* reference: panic in OpGuards::check_dtypes (ops/matmul.rs:454-477) */
    RT_ERR_INVARIANT = 3,   /* reference: panic in Matmul::new / GEMMSpec::new (ops/matmul.rs:258-282, 67-94) */
    RT_ERR_ARG = 4,         /* null pointer, bad enum, size mismatch */
    RT_ERR_CUDA = 5,        /* a CUDA runtime call failed; message holds cudaGetErrorString */
    RT_ERR_UNSUPPORTED = 6, /* legal request this build has no kernel for */
    RT_ERR_NOMEM = 7,
    RT_ERR_COMM = 8,        /* NCCL failure in the sharded path */
    RT_ERR_COMM_TIMEOUT = 9
} rt_status;

/* crates/ratchet-core/src/dtype/mod.rs:10-20 (DType).  RT_BF16 as a matmul operand and
 * RT_Q4_K are extensions the reference declares but does not implement
 * (dtype/mod.rs:12, crates/ratchet-loader/src/k_quants.rs:95-103).
 * Values outside the ordinary: an infinite or NaN activation gives what the product has by
 * IEEE's rules (+-inf by the weight's sign, NaN against a zero weight or for a NaN) in its own
 * output row and touches no other row, on every route; bf16 activations of any magnitude are
 * taken as they are (against quantised weights they are brought into f16's range row by row
 * with a power of two that is multiplied back onto the accumulator). */
typedef enum rt_dtype {
    RT_F32 = 0,
    RT_F16 = 1,
    RT_BF16 = 2,
    RT_I32 = 3,
    RT_U32 = 4,
    RT_Q8_0H = 5, /* GGUF Q8_0 split into codes | f16 scales */
    RT_Q8_0F = 6, /* GGUF Q8_0 split into codes | f32 scales */
    RT_Q4_K = 7   /* raw GGUF Q4_K super-blocks, 144 bytes per 256 values */
} rt_dtype;

typedef enum rt_epilogue {
    RT_EPILOGUE_NONE = 0,
    /* bias add, then the tanh GELU of crates/ratchet-core/src/ops/unary.rs:97-119 evaluated
     * in f32 on the value rounded to the output dtype, then rounded again: the chain
     * fc1 -> full() -> gelu() -> cast() of crates/ratchet-models/src/whisper/mlp.rs:18-22
     * fused into the producing kernel.  bf16 outputs (which the reference does not have) are
     * the exception: bias and GELU act on the f32 accumulator and the result is rounded once. */
    RT_EPILOGUE_GELU_TANH = 1,
    /* The gate/up form of crates/ratchet-models/src/phi3/mlp.rs:31-39, for the Linear node
     * W.gemm(x, b, false, true, true) only: W is [2*ff, K] with the gate rows first; the node's
     * output is [.., ff] (out_shape has the last extent halved) and holds
     *   up * cast(silu(full(gate)))      silu(v) = v * sigmoid(v), sigmoid as ops/unary.rs:121-131
     * where gate and up are the two halves of the plain node's row, each rounded to the output
     * dtype (bias added there) as the plain node would leave them; silu runs in f32 on the
     * rounded gate, is rounded to the output dtype, and the product is rounded once more (bf16
     * outputs, which the reference does not have, skip the rounding of silu).  The tensor-core GEMM
     * computes both halves of a column in one tile and never writes the [.., 2*ff] tensor; the
     * GEMV-shaped routes write it to plan scratch and run a second, elementwise launch. */
    RT_EPILOGUE_SILU_MUL = 2
} rt_epilogue;

typedef struct rt_shape {
    int32_t rank;
    int64_t dims[RT_MAX_RANK];
} rt_shape;

typedef struct rt_segment {
    uint64_t offset;
    uint64_t size;
} rt_segment;

/* One Matmul node: the fields of `Matmul` (ops/matmul.rs:248-255) plus the operand views. */
typedef struct rt_matmul_desc {
    rt_dtype lhs_dt;
    rt_dtype rhs_dt;
    rt_dtype bias_dt;      /* ignored unless has_bias */
    rt_shape lhs_shape;
    rt_shape rhs_shape;
    rt_shape bias_shape;   /* ignored unless has_bias; must be a vector */
    int32_t has_bias;
    int32_t trans_lhs;
    int32_t trans_rhs;
    int32_t trans_out;
    int32_t epilogue;      /* rt_epilogue; the reference has only RT_EPILOGUE_NONE */
} rt_matmul_desc;

/* What GEMMSpec exposes (ops/matmul.rs:31-245), for callers and tests. */
typedef struct rt_gemm_spec {
    rt_shape out_shape;     /* compute_c_shape */
    rt_dtype out_dt;        /* = rhs dtype (ops/matmul.rs:438) */
    int64_t lhs_stack, rhs_stack, out_stack, stacks;
    int64_t dim_lhs_outer;  /* M: rows of op(lhs) */
    int64_t dim_rhs_outer;  /* N: columns of op(rhs) */
    int64_t dim_inner;      /* K */
    int32_t is_gemv;        /* rhs is a vector and lhs is not transposed (ops/matmul.rs:221-223) */
} rt_gemm_spec;

typedef struct rt_device rt_device;
typedef struct rt_buffer rt_buffer;
typedef struct rt_plan rt_plan;
typedef struct rt_executable rt_executable;

/* ------------------------------------------------------------------ errors, version */

/* thiserror / anyhow messages of the reference (ops/op.rs:131-144, tensor.rs:26-38). */
const char *rt_last_error(void);
const char *rt_status_name(rt_status s);
/* "ratchet_b200 <semver> sm_100a"; lets a binding check what it loaded. */
const char *rt_version(void);
/* sizeof / offsetof of the public structs above and below, in the order the implementation
 * documents (api.cu), so that a binding can check its mirror of them; returns the entry count. */
int32_t rt_abi_layout(uint64_t *out, int32_t n);

/* ------------------------------------------------------------------ dtypes and layouts (host) */

/* DType::size_of for the plain types (dtype/mod.rs:54-64); 0 for block formats. */
size_t rt_dtype_size(rt_dtype dt);
int32_t rt_dtype_is_quantized(rt_dtype dt);          /* dtype/mod.rs:66-68 */
rt_status rt_dtype_activation(rt_dtype dt, rt_dtype *out); /* dtype/mod.rs:77-83 */

/* DType::segments (dtype/mod.rs:85-95) / Q8_0<T>::segments (dtype/blocks.rs:61-74):
 * the byte ranges of one tensor's buffer.  Q8_0: codes then scales, each padded to 256 B.
 * Plain types: one segment of max(numel*size, 16) rounded up to 4 B.  Q4_K: one segment of
 * numel/256*144 bytes.  `segs` has room for *n_segs entries; *n_segs is set to the count. */
rt_status rt_dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int32_t *n_segs);
/* Sum of the segment sizes: the bytes a tensor of this dtype occupies on the device. */
rt_status rt_dtype_nbytes(rt_dtype dt, uint64_t numel, uint64_t *nbytes);

/* Quantizer::sint8_quantize (quant.rs:26-79): f32 -> Q8_0F buffer; with RT_Q8_0H the same
 * codes with the scale rounded to f16 (what the loader holds, gguf/dtype.rs:80-109).
 * `out` must hold rt_dtype_nbytes(dt, numel).  numel % 32 == 0. */
rt_status rt_quantize_q8_0(const float *src, uint64_t numel, rt_dtype dt, void *out);
/* Quantizer::sint8_dequantize (quant.rs:81-124): (i8)q * d in f32; for RT_Q8_0H the f16
 * product f16(q)*d widened to f32. */
rt_status rt_dequantize_q8_0(const void *src, uint64_t numel, rt_dtype dt, float *out);
/* GGUFInterop::transcode for Q8_0H / Q8_0F (crates/ratchet-loader/src/gguf/dtype.rs:44-110):
 * n_blocks GGUF blocks {f16 d; i8 qs[32]} -> codes | pad | scales | pad. */
rt_status rt_transcode_gguf_q8_0(const void *blocks, uint64_t n_blocks, rt_dtype dt, void *out);
/* Q4_K encode / decode of raw GGUF super-blocks (format: k_quants.rs:95-103; no reference
 * counterpart for the arithmetic, which follows the published GGUF format). */
rt_status rt_quantize_q4_k(const float *src, uint64_t numel, void *out);
rt_status rt_dequantize_q4_k(const void *src, uint64_t numel, float *out);

/* ------------------------------------------------------------------ Matmul rules (host) */

/* Matmul::new guards + OpGuards::check_dtypes + compute_c_shape + GEMMSpec::new
 * (ops/matmul.rs:258-361, 442-478, 53-134).  Fills *spec on success. */
rt_status rt_matmul_spec(const rt_matmul_desc *desc, rt_gemm_spec *spec);
/* Matmul::compute_c_shape alone (ops/matmul.rs:284-361). */
rt_status rt_matmul_out_shape(const rt_matmul_desc *desc, rt_shape *out);

/* ------------------------------------------------------------------ device and storage */

/* Device::request_device(DeviceRequest::GPU) / WgpuDevice::new
 * (crates/ratchet-core/src/device.rs:71-80, gpu/device.rs:47-118): one CUDA device + one
 * stream.  Fails with RT_ERR_CUDA when no sm_100 device is present: there is no CPU path. */
rt_status rt_device_create(int32_t ordinal, rt_device **dev);
rt_status rt_device_destroy(rt_device *dev);
/* device.poll(WaitForSubmissionIndex) (tensor.rs:785): wait for the device's stream. */
rt_status rt_device_sync(rt_device *dev);
/* The device's cudaStream_t, as a void*. */
void *rt_device_stream(rt_device *dev);
int32_t rt_device_sm_count(rt_device *dev);
/* The CUDA ordinal the device was created with (gpu/device.rs:105 keeps `ordinal` too). */
int32_t rt_device_ordinal(rt_device *dev);

/* GPUBuffer::from_bytes / BufferPool allocation (storage/gpu_buffer.rs:46-61,
 * gpu/pools/buffer_pool.rs:82-95): sizes are rounded up to 4 B, minimum 16 B.  A freed block
 * goes back to the device's pool and may be handed out again at once: that is safe for work
 * queued on the device's own stream (it runs in order); work on other streams that still uses
 * the block must have finished before rt_buffer_free. */
rt_status rt_buffer_alloc(rt_device *dev, uint64_t nbytes, rt_buffer **buf);
rt_status rt_buffer_free(rt_buffer *buf);
void *rt_buffer_ptr(rt_buffer *buf);
uint64_t rt_buffer_size(rt_buffer *buf);
/* queue.write_buffer + submit (gpu_buffer.rs:51-61) and DownloadBuffer (gpu_buffer.rs:155-178).
 * Both are ordered on the device's stream; `sync` != 0 waits for completion.  For a copy to
 * overlap anything the host memory must be page-locked (rt_host_alloc). */
rt_status rt_upload(rt_device *dev, rt_buffer *dst, uint64_t dst_off, const void *host, uint64_t n, int32_t sync);
rt_status rt_download(rt_device *dev, const rt_buffer *src, uint64_t src_off, void *host, uint64_t n, int32_t sync);
/* Page-locked host memory for the two calls above. */
rt_status rt_host_alloc(uint64_t nbytes, void **ptr);
rt_status rt_host_free(void *ptr);

/* ------------------------------------------------------------------ compile + dispatch */

/* MetaOperation::compile for Matmul (op.rs:304-362, ops/matmul.rs:480-647): validates the
 * node, routes GEMV vs GEMM (ops/matmul.rs:540-592), picks the kernel and its launch shape
 * and allocates whatever scratch the kernel needs.  Equal descriptions on one device share one
 * plan (the role of the KernelKey lookup, ops/matmul.rs:485-524, op.rs:169-196): the device keeps
 * a cache, the call is thread-safe, and rt_plan_destroy only gives the caller's hold back.
 * A plan may be launched any number of times, with these limits: it owns ONE scratch area
 * (dequantised weights, transposed or padded operands, the f32 pre-split, partial sums), so only
 * one launch of a plan may be in flight at a time unless its launches are ordered on one stream;
 * two streams, or two graphs replayed concurrently, that launch the same plan race on it. */
rt_status rt_matmul_plan(rt_device *dev, const rt_matmul_desc *desc, rt_plan **plan);
rt_status rt_plan_destroy(rt_plan *plan);
/* Drops the dequantised copies a plan keeps of weights launched with RT_LAUNCH_LHS_CONSTANT (see
 * there).  rt_buffer_free does this by itself for buffers of this library; call it before reusing
 * the memory of a weight that came from another allocator. */
rt_status rt_plan_forget_weights(rt_plan *plan);
/* GEMMSpec of the planned node. */
rt_status rt_plan_spec(const rt_plan *plan, rt_gemm_spec *spec);
/* Name of the kernel the plan launches (the role of KernelKey, ops/matmul.rs:485-524). */
const char *rt_plan_kernel(const rt_plan *plan);
/* Number of kernel launches one rt_matmul_launch issues. */
int32_t rt_plan_launches(const rt_plan *plan);

/* CompiledOp dispatch (compiled_op.rs:13-19, executable.rs:25-54): enqueue the node on
 * `stream` (a cudaStream_t; NULL = the device's stream).  Asynchronous.  `lhs`, `rhs`,
 * `bias` are read-only device pointers to buffers laid out as rt_dtype_segments says;
 * `out` must not alias them and holds rt_dtype_nbytes(spec.out_dt, numel(out_shape)). */
rt_status rt_matmul_launch(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream);

/* Launch options.
 * RT_LAUNCH_LHS_CONSTANT: the caller states that no work in flight on the stream writes the lhs
 * bytes (a weight uploaded earlier: the leaf tensors of the reference's graph, tensor.rs:589-599).
 * A kernel may then request the weights before it waits for its stream predecessor (programmatic
 * dependent launch), which overlaps one layer's weight streaming with the previous layer's tail.
 * A tensor-core GEMM over block-format weights also keeps the weight's dequantised f16 copy with
 * the plan, keyed by the lhs pointer (2 bytes per weight of device memory, allocated at the first
 * launch with that weight: make that launch outside any stream capture): later launches skip the
 * dequantising pass.  The copy is filled on the stream of that first launch; launches on other
 * streams must be ordered after it.  RT_KEEP_WEIGHTS=0 in the environment turns this off.
 * Never set the flag for an lhs that an earlier node of the same stream produces (attention scores). */
#define RT_LAUNCH_LHS_CONSTANT 1u
/* n_out > 0 places the result somewhere else than `out`: element (r, s) of the node's [R][S]
 * output goes to outs[d][r*out_ld + out_col + s] for every d < n_out.  This is the N-sharded
 * prefill form (no reference counterpart: the reference is single-device, gpu/device.rs:15-16):
 * each GPU computes the column slice of its weight shard and writes it into every GPU's
 * full-width [rows][N] output through peer-mapped pointers (rt_ipc_open), so no separate
 * all-gather runs.  Only the tensor-core GEMM takes it (RT_ERR_UNSUPPORTED otherwise), with
 * trans_out set and one shared weight.  The caller synchronises all GPUs before reading. */
typedef struct rt_launch_opts {
    uint32_t flags;
    int32_t n_out;
    void *outs[RT_MAX_PEERS];
    int64_t out_ld;
    int64_t out_col;
} rt_launch_opts;
/* rt_matmul_launch with options; opts may be NULL. */
rt_status rt_matmul_launch_ex(rt_plan *plan, const void *lhs, const void *rhs, const void *bias, void *out, void *stream,
                              const rt_launch_opts *opts);

/* One dispatch: the operands of one planned node. */
typedef struct rt_dispatch {
    rt_plan *plan;
    const void *lhs;
    const void *rhs;
    const void *bias; /* NULL when the node has no bias */
    void *out;
    rt_launch_opts opts;
} rt_dispatch;

/* Executable (executable.rs:13-54): an ordered list of compiled nodes with their buffers bound,
 * dispatched in one call in list order on one stream (the reference records them into one
 * compute pass and submits once).  With `use_graph` != 0 the list is captured once into a CUDA
 * graph at creation (on a private stream; capturing executes nothing) and each dispatch is one
 * graph launch.  A list of two or more single-vector Q8_0H GEMVs whose weights are all flagged
 * RT_LAUNCH_LHS_CONSTANT, each reading its predecessor's output, becomes ONE persistent kernel
 * instead (rows are handed from node to node as tagged words that the readers poll; weights of
 * later nodes are streamed while earlier ones compute; same products as node-by-node dispatch,
 * f32 sums in another order);
 * only one dispatch of such an executable may be in flight at a time.  Plans and buffers must
 * outlive the executable. */
rt_status rt_executable_create(rt_device *dev, const rt_dispatch *nodes, int32_t n_nodes, int32_t use_graph, rt_executable **exe);
rt_status rt_executable_dispatch(rt_executable *exe, void *stream);
rt_status rt_executable_destroy(rt_executable *exe);
/* Kernel launches one dispatch issues (graph or not). */
int32_t rt_executable_launches(const rt_executable *exe);
/* How the list is dispatched: "nodes", "graph", or the persistent kernel's name. */
const char *rt_executable_kernel(const rt_executable *exe);

/* ------------------------------------------------------------------ activation planner
 * TensorUsageRecord (crates/ratchet-core/src/gpu/buffer_allocator/tensor_usage_record.rs): an
 * intermediate's size and the positions, in execution order, of the node that produces it and of
 * the last node that reads it. */
typedef struct rt_usage_record {
    uint64_t size;
    int32_t producer;
    int32_t last_consumer;
} rt_usage_record;
/* BufferAllocator::greedy_by_size (gpu/buffer_allocator/allocator.rs:209-271): records from the
 * largest to the smallest; each takes the last shared object (in creation order) none of whose
 * tenants is alive at the same time (two records are alive together when max(producers) <=
 * min(last_consumers)), else opens a new object of its own size.  objects[i] = shared object of
 * record i; the objects are laid end to end in one arena, each on an `alignment` boundary (a power
 * of two): offsets[i] = byte offset of record i's object, *arena_bytes = the arena's size.  Any of
 * the output pointers may be NULL.  Host only. */
rt_status rt_arena_plan(const rt_usage_record *records, int32_t n, uint64_t alignment, int32_t *objects,
                        uint64_t *offsets, int32_t *n_objects, uint64_t *arena_bytes);

/* Which operands of a node are intermediates of the executable: -1 = the pointer in rt_dispatch,
 * k >= 0 = intermediate k (the pointer in rt_dispatch is then ignored). */
typedef struct rt_node_tensors {
    int32_t lhs, rhs, bias, out;
} rt_node_tensors;
/* rt_executable_create for a node list whose intermediates the library places
 * (Executable + BufferAllocator::allocate_cfg, executable.rs:13-54, allocator.rs:273-340):
 * tensor_bytes[k] is the size of intermediate k; usage records are taken from the node list
 * (producer = the first node writing k, last consumer = the last node touching it), every node's
 * plan scratch is one more record alive during that node only, rt_arena_plan places them all, and
 * ONE device allocation made here holds them: dispatches allocate nothing, and executables do not
 * share scratch with each other or with direct launches of the same plans.  (Dequantised copies of
 * weights flagged RT_LAUNCH_LHS_CONSTANT stay with their plans; they are weights, not
 * activations.)  An intermediate must be produced by an earlier node than any that reads it
 * (RT_ERR_ARG) and be large enough for its producer's output.  `ids` may be NULL: then only the
 * plan scratch is placed.  rt_executable_create is this call with ids = NULL. */
rt_status rt_executable_create_planned(rt_device *dev, const rt_dispatch *nodes, const rt_node_tensors *ids, int32_t n_nodes,
                                       const uint64_t *tensor_bytes, int32_t n_tensors, int32_t use_graph,
                                       rt_executable **exe);
/* The executable's arena: its size, the number of shared objects in it and the sum of all its
 * records' sizes (what separate allocations would have taken).  Any pointer may be NULL. */
rt_status rt_executable_arena(const rt_executable *exe, uint64_t *arena_bytes, int32_t *n_objects, uint64_t *record_bytes);
/* Device address of intermediate `id` (NULL when out of range): valid while the executable lives;
 * its contents are defined only between its producer and its last consumer. */
void *rt_executable_tensor(const rt_executable *exe, int32_t id);

/* The MLP block as one executable (Module::schedule of crates/ratchet-models/src/phi2/mlp.rs:13-15,
 * whisper/mlp.rs:18-22, phi3/mlp.rs:31-39): hidden = act(fc1(x)), out = fc2(hidden), where fc1's
 * description carries the activation as its epilogue (RT_EPILOGUE_GELU_TANH: Phi-2 / Whisper /
 * Moondream; RT_EPILOGUE_SILU_MUL: Phi-3, fc1 being the gate_up projection) and both are Linear
 * nodes (trans_rhs, trans_out).  fc1's output shape must be fc2's rhs shape.  The hidden tensor is
 * an intermediate placed by the planner; weights are taken as constant (RT_LAUNCH_LHS_CONSTANT).
 * One row against Q8_0H weights becomes the persistent GEMV kernel over both nodes. */
typedef struct rt_mlp_desc {
    rt_matmul_desc fc1, fc2;
    const void *w1, *b1; /* b1 / b2 NULL when the description has no bias */
    const void *w2, *b2;
    const void *x;
    void *out;
} rt_mlp_desc;
rt_status rt_mlp_create(rt_device *dev, const rt_mlp_desc *mlp, int32_t use_graph, rt_executable **exe);

/* Linear-shaped Q8_0 GEMM for callers that must not allocate device memory: out[rows][n] =
 * x[rows][k] . W[n][k]^T (+ bias[n]) (+ GELU), W as RT_Q8_0H, x / bias / out f16 -- the node
 * W.gemm(x, b, false, true, true) of nn::Linear.  It has no counterpart in the reference.
 * The dequantised weights go to an array of RT_STATIC_SCRATCH_BYTES built into the library
 * (held by every GPU that loads it until exit) instead of a per-plan cudaMalloc, so weights with
 * n*k*2 > RT_STATIC_SCRATCH_BYTES are refused with RT_ERR_UNSUPPORTED.  The first call on a
 * device looks the array's address up; make that call before any stream capture.  All calls
 * share the one array and it keeps the last call's contents: calls that may overlap on the GPU
 * (different streams, or graphs replayed concurrently) race on it and must be serialised by the
 * caller.  Nothing has to be cleared between calls.  `stream` NULL = the device's stream. */
#define RT_STATIC_SCRATCH_BYTES (8u << 20)
rt_status rt_linear_q8_0_static_scratch(rt_device *dev, const void *w, const void *x, const void *bias, void *out,
                                        int64_t rows, int64_t n, int64_t k, int32_t epilogue, void *stream);

/* ------------------------------------------------------------------ N-sharded prefill (multi-GPU)
 * No reference counterpart: the reference is single-device (gpu/device.rs:15-16).  One process per
 * GPU; W is split along N (rows of the [N,K] weight, and the bias), the activations are replicated,
 * every GPU computes out[:, n0:n1].  The slices meet either through rt_comm_all_gather (NCCL over
 * NVLink) or by launching with scattered outputs (rt_launch_opts.n_out) into peer-mapped buffers. */
typedef struct rt_comm rt_comm;
#define RT_COMM_ID_BYTES 128
#define RT_IPC_HANDLE_BYTES 64
/* ncclGetUniqueId: rank 0 creates the id and sends it to the other ranks. */
rt_status rt_comm_unique_id(void *id);
/* Joins without blocking and polls until every rank has joined or timeout_ms passed
 * (RT_ERR_COMM_TIMEOUT; 0 = 60 s). */
rt_status rt_comm_init_rank(rt_device *dev, int32_t n_ranks, int32_t rank, const void *id, int32_t timeout_ms, rt_comm **comm);
/* recv = n_ranks chunks of bytes_per_rank, chunk r = rank r's send buffer.  Asynchronous on `stream`. */
rt_status rt_comm_all_gather(rt_comm *comm, const void *send, void *recv, uint64_t bytes_per_rank, void *stream);
rt_status rt_comm_destroy(rt_comm *comm);
/* CUDA IPC: export a buffer's 64-byte handle, map a peer's buffer into this process. */
rt_status rt_ipc_export(rt_buffer *buf, void *handle);
rt_status rt_ipc_open(rt_device *dev, const void *handle, void **ptr);
rt_status rt_ipc_close(rt_device *dev, void *ptr);
/* Host: rows [r0, r1) of a [rows][k] tensor repacked in the dtype's own segment layout, i.e. an
 * ordinary tensor of shape [r1-r0][k] holding rt_dtype_nbytes(dt, (r1-r0)*k) bytes. */
rt_status rt_shard_rows(rt_dtype dt, const void *src, uint64_t rows, uint64_t k, uint64_t r0, uint64_t r1, void *dst);

/* Debug / parity helper: dequantise a device tensor into f32 (RT_Q8_0F, RT_Q4_K) or f16
 * (RT_Q8_0H) exactly as the kernels decode it, so "bit-exact dequantised weights" can be
 * checked on the device.  Arithmetic: quant.rs:114-120; gemm.rs:400-406 for the f16 form. */
rt_status rt_dequantize_device(rt_device *dev, rt_dtype dt, uint64_t numel, const void *src, void *dst, void *stream);

/* ------------------------------------------------------------------ GGUF files (weight load) */

/* The loader that feeds the Matmul its weights: crates/ratchet-loader/src/gguf/gguf.rs.
 * rt_gguf_open = Header::read (gguf.rs:409-480): magic "GGUF" in either byte order, versions
 * 1-3 (32-bit lengths in v1, 64-bit after), metadata key/values, tensor infos with the
 * dimensions REVERSED so the outermost comes first (gguf.rs:452), and the tensor data offset
 * rounded up to `general.alignment` (default 32).  Errors (RT_ERR_ARG with the reference's
 * message): unknown magic, unsupported version, unrecognized value type, a bool that is not
 * 0/1; plus, which the reference leaves to its reader, any length that runs past the end of
 * the file.  A ggml type id outside lib.rs:57-80 is RT_ERR_DTYPE. */
typedef struct rt_gguf rt_gguf;

/* gguf.rs:183-216 (ValueType); the numbers are the file's. */
typedef enum rt_gguf_type {
    RT_GGUF_U8 = 0, RT_GGUF_I8 = 1, RT_GGUF_U16 = 2, RT_GGUF_I16 = 3, RT_GGUF_U32 = 4,
    RT_GGUF_I32 = 5, RT_GGUF_F32 = 6, RT_GGUF_BOOL = 7, RT_GGUF_STRING = 8, RT_GGUF_ARRAY = 9,
    RT_GGUF_U64 = 10, RT_GGUF_I64 = 11, RT_GGUF_F64 = 12
} rt_gguf_type;

/* gguf.rs:218-232 (Value), flattened for C.  Integers and bools fill u64, i64 and f64 alike;
 * floats fill f64 only.  `str` (strings; NUL-terminated, trailing NULs of the file dropped as
 * in read_string, gguf.rs:165-180) and `node` stay valid until rt_gguf_close. */
typedef struct rt_gguf_value {
    int32_t type;       /* rt_gguf_type */
    int32_t elem_type;  /* arrays: the elements' rt_gguf_type; else -1 */
    uint64_t len;       /* strings: bytes; arrays: elements; else 1 */
    uint64_t u64;
    int64_t i64;
    double f64;
    const char *str;
    const void *node;   /* opaque; what rt_gguf_array_item walks */
} rt_gguf_value;

/* gguf.rs:56-60 (TensorInfo) plus size_in_bytes (93-98). */
typedef struct rt_gguf_tensor_info {
    const char *name;   /* valid until rt_gguf_close */
    uint32_t ggml_type; /* lib.rs:57-80: 0 F32, 1 F16, 8 Q8_0, 12 Q4_K, ... */
    rt_shape shape;     /* outermost first */
    uint64_t offset;    /* from the start of the tensor data */
    uint64_t nbytes;    /* numel / block_numel * type_size */
} rt_gguf_tensor_info;

rt_status rt_gguf_open(const char *path, rt_gguf **out);
rt_status rt_gguf_close(rt_gguf *g);
int32_t rt_gguf_version(const rt_gguf *g);
uint64_t rt_gguf_alignment(const rt_gguf *g);
uint64_t rt_gguf_tensor_data_offset(const rt_gguf *g);   /* Header::tensor_data_offset */
uint64_t rt_gguf_tensor_count(const rt_gguf *g);
uint64_t rt_gguf_metadata_count(const rt_gguf *g);
/* Entries in file order.  rt_gguf_metadata_find = Metadata::get (gguf.rs:149-153): an absent
 * key is RT_ERR_ARG "missing key <key>". */
rt_status rt_gguf_metadata_at(const rt_gguf *g, uint64_t index, const char **key, rt_gguf_value *value);
rt_status rt_gguf_metadata_find(const rt_gguf *g, const char *key, rt_gguf_value *value);
rt_status rt_gguf_array_item(const rt_gguf_value *array, uint64_t index, rt_gguf_value *item);
/* An absent name is RT_ERR_ARG "cannot find tensor info for <name>" (gguf.rs:490-493). */
rt_status rt_gguf_tensor_at(const rt_gguf *g, uint64_t index, rt_gguf_tensor_info *info);
rt_status rt_gguf_tensor_find(const rt_gguf *g, const char *name, rt_gguf_tensor_info *info);
/* ratchet_from_gguf (gguf.rs:113-141): the dtype a tensor loads as.  F32 and F16 as they are;
 * Q8_0 as RT_Q8_0H (the f16-capable-device branch, gguf.rs:130-136; RT_Q8_0F may be asked for
 * instead); Q4_K as RT_Q4_K (extension: the reference rejects it); every other ggml type is
 * RT_ERR_UNSUPPORTED "unsupported ggml dtype". */
rt_status rt_gguf_tensor_dtype(const rt_gguf *g, const char *name, rt_dtype *dt);
/* TensorInfo::read (gguf.rs:62-84) + GGUFInterop::transcode (gguf/dtype.rs:44-110) on the host:
 * writes the tensor in the device layout of `dt` (rt_dtype_segments) to `out`.  RT_ERR_SHAPE when
 * the element count does not divide by the block size, RT_ERR_DTYPE when the tensor cannot load
 * as `dt`. */
rt_status rt_gguf_read_tensor(rt_gguf *g, const char *name, rt_dtype dt, void *out, uint64_t out_bytes);
/* The same checks without reading: the bytes rt_gguf_read_tensor would write. */
rt_status rt_gguf_tensor_nbytes(const rt_gguf *g, const char *name, rt_dtype dt, uint64_t *nbytes);
/* The same, uploaded into a new device buffer (freed by the caller); *shape may be NULL. */
rt_status rt_gguf_load_tensor(rt_gguf *g, rt_device *dev, const char *name, rt_dtype dt, rt_buffer **buf, rt_shape *shape);

#ifdef __cplusplus
}
#endif
#endif /* RATCHET_B200_H */
