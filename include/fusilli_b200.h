/*
 * fusilli_b200.h -- C ABI of libfusilli_b200.so, the B200 (sm_100a) execution
 * backend that sits under the Fusilli graph API.
 *
 * The reference reaches its compute through two foreign interfaces: the IREE
 * compiler C API (graph text -> compiled module bytes,
 * include/fusilli/backend/compile_session.h:337-371, :489-570) and the IREE
 * runtime C API (device, buffer views, module load, invoke,
 * include/fusilli/backend/runtime.h:81-674). Every function below names the
 * reference call site it stands in for. Only plain C types cross this
 * boundary: pointers, sizes, fixed-width integers and POD structs.
 *
 * Conventions
 *  - every call returns an fb_status; 0 is success. The numeric values are the
 *    reference's ErrorCode values (include/fusilli/support/logging.h:58-71) so
 *    the C++ host maps them 1:1.
 *  - fb_last_error() returns the message of the last failing call made by the
 *    calling thread (thread local, valid until that thread's next fb_* call).
 *  - launches are asynchronous on the device's stream; fb_buffer_d2h and
 *    fb_device_sync are the synchronisation points, as Buffer::read is in the
 *    reference (include/fusilli/graph/graph.h:209-241).
 *  - there is no CPU execution path in this library. Without a usable CUDA
 *    device every device/buffer/plan-load/execute call fails with
 *    FB_RUNTIME_FAILURE; only fb_plan_build (pure host lowering) works.
 */
#ifndef FUSILLI_B200_H
#define FUSILLI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_ABI_VERSION 3
#define FB_MAX_RANK 8
#define FB_MAX_NODE_INPUTS 6
#define FB_MAX_NODE_OUTPUTS 3

/* Status codes: same numbering as fusilli::ErrorCode (logging.h:58-71). */
typedef int32_t fb_status;
enum {
  FB_OK = 0,
  FB_NOT_IMPLEMENTED = 1,
  FB_NOT_VALIDATED = 2,
  FB_NOT_COMPILED = 3,
  FB_ATTRIBUTE_NOT_SET = 4,
  FB_INTERNAL_ERROR = 5,
  FB_INVALID_ATTRIBUTE = 6,
  FB_INVALID_ARGUMENT = 7,
  FB_VARIANT_PACK_ERROR = 8,
  FB_COMPILE_FAILURE = 9,
  FB_RUNTIME_FAILURE = 10,
  FB_FILE_SYSTEM_FAILURE = 11
};

/* Element types: same numbering as fusilli::DataType
 * (include/fusilli/attributes/types.h:27-47). */
enum {
  FB_DT_NOT_SET = 0,
  FB_DT_HALF = 1,
  FB_DT_BFLOAT16 = 2,
  FB_DT_FLOAT = 3,
  FB_DT_DOUBLE = 4,
  FB_DT_UINT8 = 5,
  FB_DT_INT4 = 6,
  FB_DT_INT8 = 7,
  FB_DT_INT16 = 8,
  FB_DT_INT32 = 9,
  FB_DT_INT64 = 10,
  FB_DT_BOOLEAN = 11,
  FB_DT_FP8E5M2 = 12
};

/* Node kinds (one per Graph builder, include/fusilli/graph/graph.h:766-1193). */
enum {
  FB_OP_CONV_FPROP = 1,
  FB_OP_CONV_DGRAD = 2,
  FB_OP_CONV_WGRAD = 3,
  FB_OP_MATMUL = 4,
  FB_OP_SDPA = 5,
  FB_OP_LAYERNORM = 6,
  FB_OP_RMSNORM = 7,
  FB_OP_REDUCTION = 8,
  FB_OP_POINTWISE = 9,
  FB_OP_BATCHNORM = 10
};

/* Pointwise modes: same order as PointwiseAttr::Mode
 * (include/fusilli/attributes/pointwise_attributes.h:27-74), NOT_SET = 0. */
enum {
  FB_PW_NOT_SET = 0,
  FB_PW_ABS,
  FB_PW_ADD,
  FB_PW_ADD_SQUARE,
  FB_PW_BINARY_SELECT,
  FB_PW_CEIL,
  FB_PW_CMP_EQ,
  FB_PW_CMP_GE,
  FB_PW_CMP_GT,
  FB_PW_CMP_LE,
  FB_PW_CMP_LT,
  FB_PW_CMP_NEQ,
  FB_PW_DIV,
  FB_PW_ELU_FWD,
  FB_PW_ERF,
  FB_PW_EXP,
  FB_PW_FLOOR,
  FB_PW_GELU_APPROX_TANH_BWD,
  FB_PW_GELU_APPROX_TANH_FWD,
  FB_PW_GELU_BWD,
  FB_PW_GELU_FWD,
  FB_PW_IDENTITY,
  FB_PW_LOG,
  FB_PW_LOGICAL_AND,
  FB_PW_LOGICAL_NOT,
  FB_PW_LOGICAL_OR,
  FB_PW_MAX_OP,
  FB_PW_MIN_OP,
  FB_PW_MUL,
  FB_PW_NEG,
  FB_PW_RECIPROCAL,
  FB_PW_RELU_BWD,
  FB_PW_RELU_FWD,
  FB_PW_RSQRT,
  FB_PW_SIGMOID_FWD,
  FB_PW_SIN,
  FB_PW_SOFTPLUS_FWD,
  FB_PW_SQRT,
  FB_PW_SUB,
  FB_PW_SWISH_BWD,
  FB_PW_SWISH_FWD,
  FB_PW_TAN,
  FB_PW_TANH_BWD,
  FB_PW_TANH_FWD,
  FB_PW_MODE_COUNT
};

/* Reduction modes: same order as ReductionAttr::Mode
 * (include/fusilli/attributes/reduction_attributes.h:27-38). */
enum {
  FB_RED_NOT_SET = 0,
  FB_RED_ADD,
  FB_RED_SUM,
  FB_RED_MUL,
  FB_RED_MIN,
  FB_RED_MAX,
  FB_RED_AMAX,
  FB_RED_AVG,
  FB_RED_NORM1,
  FB_RED_NORM2,
  FB_RED_MUL_NO_ZEROS,
  FB_RED_MODE_COUNT
};

/* Role of a tensor inside one graph. */
enum {
  FB_TENSOR_INPUT = 0,   /* graph input, bound to a buffer at execute        */
  FB_TENSOR_OUTPUT = 1,  /* non-virtual node output, bound at execute        */
  FB_TENSOR_VIRTUAL = 2, /* intermediate; lives in registers or workspace    */
  FB_TENSOR_SCALAR = 3   /* compile-time constant, never bound               */
};

/* Node flags. */
enum {
  FB_FLAG_SDPA_CAUSAL = 1,
  FB_FLAG_SDPA_GQA = 2,
  FB_FLAG_SDPA_HAS_SCALE = 4,
  FB_FLAG_NORM_TRAINING = 8
};

/* One tensor of the validated graph: logical dims plus element strides, the
 * reference's TensorAttr after inference
 * (include/fusilli/attributes/tensor_attributes.h:374-809). `arg_index` is the
 * position of the tensor's buffer in fb_plan_execute's pointer list (non-virtual
 * outputs sorted by name first, then non-scalar inputs sorted by name -- the
 * argument order of the reference's generated function,
 * include/fusilli/backend/runtime.h:426-457); -1 for virtual and scalar.
 * Bit k of `dynamic_mask` marks logical dim k as dynamic
 * (TensorAttr::setDynamicDims, tensor_attributes.h:512-570): `dims` and
 * `strides` then hold the representative extent and the dense layout pattern,
 * and fb_plan_execute_shaped takes the extent of each call. */
typedef struct fb_tensor_desc {
  const char *name;
  int32_t dtype;
  int32_t role;
  int32_t rank;
  int32_t arg_index;
  int64_t dims[FB_MAX_RANK];
  int64_t strides[FB_MAX_RANK];
  double scalar_value; /* role == FB_TENSOR_SCALAR only */
  uint32_t dynamic_mask;
  int32_t reserved;
} fb_tensor_desc;

/* One node. Tensor slots by op (index into fb_graph_desc.tensors, -1 = absent):
 *   CONV_FPROP  in {X, W}              out {Y}
 *   CONV_DGRAD  in {DY, W}             out {DX}
 *   CONV_WGRAD  in {DY, X}             out {DW}
 *   MATMUL      in {A, B}              out {C}
 *   SDPA        in {Q, K, V, MASK}     out {O}
 *   LAYERNORM   in {X, SCALE, BIAS, EPSILON}  out {Y, MEAN, INV_VARIANCE}
 *   RMSNORM     in {X, SCALE, EPSILON}        out {Y}
 *   BATCHNORM   in {X, SCALE, BIAS, MEAN, VAR, EPSILON}  out {Y, SAVED_MEAN, SAVED_INV_VARIANCE}
 *               (FB_FLAG_NORM_TRAINING: batch statistics; else the running MEAN / VAR)
 *   REDUCTION   in {X}                 out {Y}
 *   POINTWISE   in {IN_0, IN_1, IN_2}  out {OUT_0}
 * fparams by op:
 *   POINTWISE   {elu_alpha, softplus_beta, softplus_threshold, swish_beta}
 *   SDPA        {scale (valid with FB_FLAG_SDPA_HAS_SCALE), dropout_p}
 *   BATCHNORM   {momentum} (carried for the record: the op is functional, as
 *               torch.aten.native_batch_norm on value tensors, and returns no
 *               updated running statistics) */
typedef struct fb_node_desc {
  const char *name;
  int32_t op;
  int32_t mode; /* FB_PW_* or FB_RED_* */
  int32_t flags;
  int32_t num_spatial; /* conv only: 1..3 */
  int32_t inputs[FB_MAX_NODE_INPUTS];
  int32_t outputs[FB_MAX_NODE_OUTPUTS];
  int32_t reserved;
  int64_t padding[3];
  int64_t stride[3];
  int64_t dilation[3];
  float fparams[4];
} fb_node_desc;

typedef struct fb_graph_desc {
  const char *name;
  int32_t num_tensors;
  int32_t num_nodes; /* in topological order, as the builders appended them */
  const fb_tensor_desc *tensors;
  const fb_node_desc *nodes;
} fb_graph_desc;

typedef struct fb_device fb_device;
typedef struct fb_buffer fb_buffer;
typedef struct fb_plan fb_plan;

/* ---- library ---------------------------------------------------------- */

/* ABI version of the loaded library (FB_ABI_VERSION it was built with). */
int32_t fb_abi_version(void);
/* Message of the calling thread's last failing fb_* call ("" if none). */
const char *fb_last_error(void);
/* Number of CUDA devices visible; 0 when there is no usable driver/GPU. */
int32_t fb_device_count(void);

/* ---- device: replaces Handle::create -> createAMDGPUDevice(deviceId, stream)
 *      (include/fusilli/backend/handle.h:40-112, runtime.h:183-231) --------- */

/* Opens device `ordinal`. `ext_stream` is a cudaStream_t to run on (borrowed,
 * never destroyed) or NULL to create and own a non-blocking stream. Thread
 * safe. Fails with FB_RUNTIME_FAILURE when the ordinal does not exist or the
 * device is not compute capability 10.x. */
fb_status fb_device_open(int32_t ordinal, void *ext_stream, fb_device **out);
fb_status fb_device_close(fb_device *dev);
/* Blocks until all work queued on the device's stream is done. */
fb_status fb_device_sync(fb_device *dev);
/* The cudaStream_t the device launches on. */
void *fb_device_stream(fb_device *dev);
int32_t fb_device_ordinal(fb_device *dev);

/* ---- buffers: replace Buffer::allocate / allocateRaw / import / read
 *      (include/fusilli/backend/runtime.h:532-674) ------------------------- */

/* Device allocation of `bytes` (> 0), stream ordered on the device's stream. */
fb_status fb_buffer_alloc(fb_device *dev, size_t bytes, fb_buffer **out);
/* Wraps caller-owned device memory (Buffer::import): never freed here. */
fb_status fb_buffer_wrap(fb_device *dev, void *dptr, size_t bytes,
                         fb_buffer **out);
fb_status fb_buffer_retain(fb_buffer *buf);
/* Drops one reference; the last one frees an owned allocation. */
fb_status fb_buffer_release(fb_buffer *buf);
/* Stream-ordered host->device copy of `bytes` from `src` (pageable or pinned);
 * returns after the source has been consumed. */
fb_status fb_buffer_h2d(fb_device *dev, fb_buffer *buf, const void *src,
                        size_t bytes);
/* Device->host copy; synchronises the stream before returning. */
fb_status fb_buffer_d2h(fb_device *dev, fb_buffer *buf, void *dst,
                        size_t bytes);
void *fb_buffer_ptr(fb_buffer *buf);
size_t fb_buffer_size(fb_buffer *buf);

/* ---- plan: replaces CompileSession::compile (graph -> artifact bytes,
 *      compile_session.h:489-570), Graph::createVmContext (artifact -> loaded
 *      module, runtime.h:242-315), Graph::queryTransientSize (runtime.h:339)
 *      and iree_vm_invoke in Graph::execute (runtime.h:524-526) ------------- */

/* Lowers a validated graph to a kernel plan and serialises it. Needs no
 * device, like Graph::compileToArtifact (graph.h:149-166). Graph patterns the
 * kernels cannot run are rejected here with FB_NOT_IMPLEMENTED, never at
 * execute. The returned bytes are owned by the caller; free with
 * fb_bytes_free. */
fb_status fb_plan_build(const fb_graph_desc *graph, uint8_t **bytes,
                        size_t *num_bytes);
void fb_bytes_free(uint8_t *bytes);
/* Deserialises artifact bytes for `dev` (copies them). Rejects a bad magic,
 * ABI version, architecture tag or truncated payload with FB_RUNTIME_FAILURE. */
fb_status fb_plan_load(fb_device *dev, const uint8_t *bytes, size_t num_bytes,
                       fb_plan **out);
fb_status fb_plan_free(fb_plan *plan);
/* Validates artifact bytes (magic, ABI version, architecture, length, checksum,
 * payload structure) without a device; the checks fb_plan_load applies. */
fb_status fb_plan_check(const uint8_t *bytes, size_t num_bytes);
/* Scratch bytes fb_plan_execute needs (0 when every intermediate is fused). */
fb_status fb_plan_workspace_size(fb_plan *plan, size_t *bytes);
/* Number of buffers fb_plan_execute expects in `args`. */
fb_status fb_plan_num_args(fb_plan *plan, int32_t *num_args);
/* Number of kernel launches one execute issues (the "dispatch-count" of the
 * reference's compile statistics). */
fb_status fb_plan_num_launches(fb_plan *plan, int32_t *num_launches);
/* Writes a NUL-terminated JSON description of the plan (steps, kernels,
 * dispatch-count, transient-memory-size) into `buf`; `*needed` receives the
 * size including the NUL. Call with cap = 0 to query. */
fb_status fb_plan_stats_json(fb_plan *plan, char *buf, size_t cap,
                             size_t *needed);
/* Enqueues the plan on the device's stream. `args[i]` is the device pointer of
 * the tensor whose arg_index is i, dense in its physical (stride) order;
 * `arg_bytes[i]` its size, checked against the plan. `workspace` may be NULL
 * when the plan needs none. Does not synchronise. */
fb_status fb_plan_execute(fb_plan *plan, fb_device *dev, void *const *args,
                          const size_t *arg_bytes, int32_t num_args,
                          void *workspace, size_t workspace_bytes);
/* fb_plan_execute for a plan whose graph has dynamic dims. `arg_dims` holds
 * FB_MAX_RANK logical extents per buffer (row i = the tensor whose arg_index
 * is i; entries past the tensor's rank are ignored): static dims must equal
 * the plan's, dynamic ones give this call's extent. The extents of virtual
 * tensors follow from the nodes' shape rules, strides are regenerated as the
 * dense layout the representative strides describe, and the kernels are chosen
 * again for the concrete shape; the result is kept in the plan, keyed by the
 * extents, so a repeated shape costs a lookup. Extents that the inputs do not
 * imply (an output buffer of the wrong shape) are FB_INVALID_ARGUMENT. The
 * workspace must cover the concrete shape; fb_plan_workspace_size reports the
 * size for the representative extents (the reference likewise has no
 * runtime-sized workspace query, runtime.h:361-369). A plan without dynamic
 * dims accepts only its own dims. */
fb_status fb_plan_execute_shaped(fb_plan *plan, fb_device *dev,
                                 void *const *args, const size_t *arg_bytes,
                                 const int64_t *arg_dims, int32_t num_args,
                                 void *workspace, size_t workspace_bytes);
/* The same specialisation without a device: artifact bytes in, artifact bytes
 * for the given extents out (free with fb_bytes_free). The result equals what
 * fb_plan_build gives for a graph declared with those extents as its
 * representative dims. */
fb_status fb_plan_specialize(const uint8_t *bytes, size_t num_bytes,
                             const int64_t *arg_dims, int32_t num_args,
                             uint8_t **out_bytes, size_t *out_num_bytes);
/* Scratch bytes fb_plan_execute_shaped needs for the given extents. */
fb_status fb_plan_workspace_size_shaped(fb_plan *plan, const int64_t *arg_dims,
                                        int32_t num_args, size_t *bytes);
/* Error word written by kernels whose bounded waits ran out (0 = none). Reads
 * it with a stream synchronise. */
fb_status fb_device_kernel_error(fb_device *dev, uint32_t *error_word);

/* Test hook for the bounded waits: launches a one-CTA kernel that waits, with a limit of
 * `spins` polls, on an mbarrier nothing ever arrives at, then returns normally. The wait runs
 * out, the kernel ORs `code` into the device's error word and ends; the context stays usable.
 * This is how failure detection is exercised without faulting or hanging the GPU. */
fb_status fb_device_selftest_wait_timeout(fb_device *dev, uint32_t spins, uint32_t code);
/* Clears the device's error word (stream ordered). */
fb_status fb_device_clear_kernel_error(fb_device *dev);

/* ---- multi-GPU exchange ---------------------------------------------------
 * No counterpart in the reference, which has no multi-device code: one Handle
 * is one device (include/fusilli/backend/runtime.h:19-24, handle.h:74-112
 * `create(backend, deviceId)`). The sharded benchmark runs one process per GPU,
 * each with its own fb_device; every op shards over its outermost extent with no
 * exchange except the convolution weight gradient (benchmarks/driver.cpp:249
 * builds the graph that is sharded): per-rank fp32 partial filter gradients are
 * summed across ranks and rounded once.
 *
 * Bootstrap (the launcher moves the bytes; any transport will do):
 *   fb_comm_create        on every rank: allocates this rank's exchange buffer
 *   fb_comm_local_handle  on every rank: FB_COMM_HANDLE_BYTES describing it
 *                         (rank 0's block also carries the NCCL unique id)
 *   -- all-gather the blocks in rank order --
 *   fb_comm_connect       on every rank, collectively: maps the peers' buffers
 *                         (cudaIpc) and creates the NCCL communicator
 * All exchange calls are enqueued on the device's stream and do not synchronise
 * the host; every rank must issue the same sequence of calls. */
#define FB_COMM_MAX_RANKS 8
#define FB_COMM_HANDLE_BYTES 256
typedef struct fb_comm fb_comm;

fb_status fb_comm_create(fb_device *dev, int32_t rank, int32_t world,
                         size_t buffer_bytes /* multiple of 256 */,
                         fb_comm **out);
fb_status fb_comm_local_handle(fb_comm *comm,
                               uint8_t *block /* FB_COMM_HANDLE_BYTES */);
fb_status fb_comm_connect(fb_comm *comm,
                          const uint8_t *blocks /* world x FB_COMM_HANDLE_BYTES */);
fb_status fb_comm_close(fb_comm *comm);
/* This rank's exchange buffer (device memory, 256-byte aligned): bind weight
 * gradient outputs and read results inside it. */
void *fb_comm_buffer(fb_comm *comm);
size_t fb_comm_buffer_bytes(fb_comm *comm);
int32_t fb_comm_rank(fb_comm *comm);
int32_t fb_comm_world(fb_comm *comm);
/* Sum over ranks of the fp32 bucket at byte offset `in_offset` of every rank's
 * exchange buffer (`count` values, a multiple of 4), rounded once to `out_dtype`
 * (FB_DT_FLOAT / BFLOAT16 / HALF) and written at `out_offset` of EVERY rank's
 * buffer: one kernel per rank over peer-mapped memory (plain loads and stores
 * over NVLink, ranks added in rank order, so all ranks hold identical bits). The
 * input bucket may be rewritten, and the output read, by the next work on the
 * stream. Waits are bounded: a rank that never arrives sets the device's error
 * word instead of hanging the others. */
fb_status fb_comm_sum_fused(fb_comm *comm, size_t in_offset, size_t count,
                            size_t out_offset, int32_t out_dtype);
/* The same sum through the library route: ncclAllReduce(sum, fp32) in place on
 * `inout_f32` (any device memory), then a cast of `count` values into `out`. */
fb_status fb_comm_sum_nccl(fb_comm *comm, void *inout_f32, size_t count,
                           void *out, int32_t out_dtype);
/* Gathers every rank's slab of `bytes_per_rank` into `recv` in rank order
 * (ncclAllGather): the output all-gather of the batch-sharded ops. */
fb_status fb_comm_allgather(fb_comm *comm, const void *send, void *recv,
                            size_t bytes_per_rank);
/* Test entry point: runs the fused exchange for `world` VIRTUAL ranks in one
 * cooperative launch on one device (kernels that wait on one another are never
 * separate launches on one GPU). `buckets`: world x count fp32 (device memory);
 * `out`: world x count values of `out_dtype`, rank r's copy at r*count. */
fb_status fb_comm_selftest_emulated(fb_device *dev, int32_t world,
                                    const float *buckets, size_t count,
                                    void *out, int32_t out_dtype,
                                    int32_t repeats);

/* ---- allocation-free weight gradient -------------------------------------
 * No counterpart in the reference: its graphs always run with whatever
 * transient memory the runtime allocates for them.
 *
 * DW = conv weight gradient of dense channels-last tensors (dy NHWC
 * [n,oh,ow,k], x NHWC [n,h,w,c], dw KRSC [k,r,s,c/groups], all of `dtype` =
 * FB_DT_HALF / FB_DT_BFLOAT16 / FB_DT_FLOAT, fp32 accumulation), for callers
 * that must not allocate when they need it: code running inside a framework's
 * allocator hook or under its allocator lock, a latency-critical loop with a
 * no-allocation rule, a plugin that only ever receives raw device pointers and a
 * stream. It takes no fb_device (opening one allocates) and calls no
 * cudaMalloc/cudaFree or allocating library routine; the partial sums of its
 * split reduction live in a fixed array of fb_conv_wgrad_static_scratch_bytes()
 * (8 MiB) inside the library image, resident on every GPU that loads the library
 * until the process exits.
 *
 *  - runs on the CURRENT device, on `stream` (a cudaStream_t, may be NULL);
 *  - the first call on each device resolves the array's device address and reads
 *    the SM count; the CUDA runtime may load this library's device code onto
 *    that GPU at that point, which can allocate. Make that first call (any valid
 *    small problem will do) during set-up: outside the region where allocation
 *    is forbidden, and before starting any stream capture on that device;
 *  - fails with FB_INVALID_ARGUMENT when k*(c/groups)*r*s fp32 values do not fit
 *    in the array -- use a plan with a caller-provided workspace for those;
 *  - all calls on a device share the one array: two calls whose kernels can
 *    overlap on the GPU (different streams, no ordering between them) race.
 *    Calls on the same stream are safe back to back; the array's old contents
 *    are never read. */
size_t fb_conv_wgrad_static_scratch_bytes(void);
fb_status fb_conv_wgrad_static(void *stream, const void *dy, const void *x,
                               void *dw, int32_t dtype, int32_t n, int32_t c,
                               int32_t h, int32_t w, int32_t k, int32_t r,
                               int32_t s, int32_t pad_h, int32_t pad_w,
                               int32_t stride_h, int32_t stride_w,
                               int32_t dil_h, int32_t dil_w, int32_t groups);

#ifdef __cplusplus
}
#endif
#endif /* FUSILLI_B200_H */
