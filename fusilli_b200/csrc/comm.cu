// Multi-GPU exchange of the sharded hot path: one fb_comm per rank (one process per GPU).
//
// Every benchmarked op shards over its outermost extent with no data-path exchange, except the
// convolution weight gradient: each rank reduces over its own images and the fp32 partial filter
// gradients have to be summed across ranks before the one rounding to the gradient's type. Two
// implementations of that sum live here:
//
//  * fb_comm_sum_nccl: ncclAllReduce(sum, fp32) in place on the caller's bucket, then one cast
//    kernel. NCCL is loaded at run time (dlopen of libnccl.so.2; inside a PyTorch process that is
//    the copy PyTorch already loaded), so the library has no link-time dependency on it.
//
//  * fb_comm_sum_fused: ONE kernel per rank over peer-mapped memory (cudaIpc), two-shot:
//      arrive    every rank publishes "my fp32 bucket is complete" in every peer's flag row and
//                waits for the same word from all peers;
//      reduce    rank r owns elements [r*chunk, (r+1)*chunk): it loads that chunk from every
//                rank's bucket with plain 16-byte ld.volatile.global over NVLink, adds them in
//                rank order 0..W-1 (so the sum does not depend on timing), rounds ONCE to the
//                output type and stores the rounded chunk into every rank's output bucket
//                (plain peer stores);
//      done      a device-wide count of finished CTAs lets the last one publish "my chunk has
//                landed everywhere"; block 0 waits for that word from all peers before the
//                kernel ends, so the next kernel on the stream sees the whole output.
//    NVLink traffic per rank: (W-1)/W of the bucket in fp32 inbound, the same in the 16-bit output
//    type outbound -- against (W-1) x the bucket for a one-shot read-everything sum. No TMA, no
//    bulk copy and no multicast touch peer memory: loads and stores only.
//    Every wait is bounded (about a second); on expiry the waiter ORs a code into the device's
//    error word (fb_device_kernel_error) and the kernel runs to its end instead of hanging.
//
// fb_comm_selftest_emulated runs the same kernel for W virtual ranks inside ONE cooperative launch
// on one GPU (blockIdx.y = rank, every rank's region in local memory), which is how the protocol
// is tested where only one GPU is available: kernels that wait on one another must never be
// separate launches on one GPU.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>

#include "common.h"

using namespace fb;

namespace {

constexpr int kMaxRanks = FB_COMM_MAX_RANKS;
constexpr size_t kHeaderBytes = 1024; // flag rows and the CTA counter, ahead of the data
constexpr uint32_t kFlagSpins = 1u << 21; // x (200 ns sleep + one load): a second or two

enum : uint32_t { ERR_COMM_ARRIVE = 0x100, ERR_COMM_DONE = 0x200 };

// ---- NCCL through dlopen ---------------------------------------------------------------
struct NcclId { char internal[128]; };
typedef void *NcclComm;
struct NcclApi {
  int (*GetUniqueId)(NcclId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
  std::string why;
};
constexpr int kNcclInt8 = 0, kNcclFloat32 = 7, kNcclSum = 0; // ncclDataType_t / ncclRedOp_t values

NcclApi &nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD); // the copy the host process loaded
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      api.why = "libnccl.so.2 not found";
      return;
    }
    auto sym = [&](const char *name) { return dlsym(h, name); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather &&
             api.GetErrorString;
    if (!api.ok) api.why = "libnccl.so.2 lacks an expected symbol";
  });
  return api;
}

#define FB_NCCL_OK(expr)                                                                           \
  do {                                                                                             \
    int _r = (expr);                                                                               \
    if (_r != 0) return fail(FB_RUNTIME_FAILURE, std::string(#expr) + ": " + nccl().GetErrorString(_r)); \
  } while (0)

// ---- the exchange kernel ---------------------------------------------------------------
struct ExchangeParams {
  int32_t world, rank0, out_dtype;
  uint32_t epoch;
  int64_t count;          // fp32 elements of the bucket (multiple of 4)
  int64_t in_off, out_off; // byte offsets of the fp32 bucket and of the output inside a region
  uint8_t *region[kMaxRanks]; // every rank's region as mapped in this process
  uint32_t *err;
};

__device__ __forceinline__ uint32_t *flag_arrive(uint8_t *region, int from) {
  return reinterpret_cast<uint32_t *>(region) + from;
}
__device__ __forceinline__ uint32_t *flag_done(uint8_t *region, int from) {
  return reinterpret_cast<uint32_t *>(region + 256) + from;
}
__device__ __forceinline__ uint32_t *cta_counter(uint8_t *region) {
  return reinterpret_cast<uint32_t *>(region + 512);
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_volatile_f4(const float4 *p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Epochs only grow; the comparison is wrap-safe.
__device__ __forceinline__ bool wait_flag(const uint32_t *p, uint32_t epoch, uint32_t *err, uint32_t code) {
  for (uint32_t it = 0; it < kFlagSpins; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - epoch) >= 0) return true;
    if (it > 64) __nanosleep(200);
  }
  if (err) atomicOr(err, code);
  return false;
}

__global__ void __launch_bounds__(512)
wgrad_exchange_kernel(const ExchangeParams p) {
  const int W = p.world;
  const int rank = p.rank0 + (int)blockIdx.y;
  uint8_t *mine = p.region[rank];

  // arrive: this rank's bucket was written by earlier kernels on this stream
  if (blockIdx.x == 0 && (int)threadIdx.x < W) st_release_sys(flag_arrive(p.region[threadIdx.x], rank), p.epoch);
  if ((int)threadIdx.x < W) wait_flag(flag_arrive(mine, threadIdx.x), p.epoch, p.err, ERR_COMM_ARRIVE);
  __syncthreads();

  // reduce this rank's chunk in rank order, round once, store into every rank's output
  const int64_t vecs = p.count / 4;
  const int64_t per = (vecs + W - 1) / W;
  const int64_t v0 = min((int64_t)rank * per, vecs), v1 = min(v0 + per, vecs);
  for (int64_t i = v0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += (int64_t)gridDim.x * blockDim.x) {
    float4 v[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < W) v[r] = ld_volatile_f4(reinterpret_cast<const float4 *>(p.region[r] + p.in_off) + i);
    float4 acc = v[0];
#pragma unroll
    for (int r = 1; r < kMaxRanks; ++r)
      if (r < W) {
        acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
      }
    if (p.out_dtype == FB_DT_FLOAT) {
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < W) reinterpret_cast<float4 *>(p.region[r] + p.out_off)[i] = acc;
    } else {
      uint2 packed;
      if (p.out_dtype == FB_DT_BFLOAT16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        packed.x = *reinterpret_cast<uint32_t *>(&lo);
        packed.y = *reinterpret_cast<uint32_t *>(&hi);
      } else {
        __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
        packed.x = *reinterpret_cast<uint32_t *>(&lo);
        packed.y = *reinterpret_cast<uint32_t *>(&hi);
      }
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < W) reinterpret_cast<uint2 *>(p.region[r] + p.out_off)[i] = packed;
    }
  }

  // done: the last CTA of this rank to finish publishes the chunk to every peer
  __syncthreads();
  __shared__ uint32_t last;
  if (threadIdx.x == 0) {
    __threadfence_system(); // this CTA's stores, before it is counted
    last = atomicAdd(cta_counter(mine), 1u) == gridDim.x - 1 ? 1u : 0u;
    __threadfence_system(); // the other CTAs' stores, before the flags below
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) *cta_counter(mine) = 0u; // every CTA has counted: ready for the next call
    if ((int)threadIdx.x < W) st_release_sys(flag_done(p.region[threadIdx.x], rank), p.epoch);
  }
  // The kernel may end only when every peer's chunk has landed in this rank's output.
  if (blockIdx.x == 0 && (int)threadIdx.x < W) wait_flag(flag_done(mine, threadIdx.x), p.epoch, p.err, ERR_COMM_DONE);
}

__global__ void __launch_bounds__(256)
cast_f32_kernel(const float *__restrict__ in, void *out, int out_dtype, int64_t count) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
    store_f(out, out_dtype, i, in[i]);
}

struct IpcBlock { // what one rank contributes to the bootstrap exchange
  cudaIpcMemHandle_t mem;
  NcclId nccl_id; // meaningful in rank 0's block only
  uint64_t region_bytes;
  uint32_t rank, has_nccl;
  uint8_t pad[FB_COMM_HANDLE_BYTES - sizeof(cudaIpcMemHandle_t) - sizeof(NcclId) - 16];
};
static_assert(sizeof(IpcBlock) == FB_COMM_HANDLE_BYTES, "bootstrap block size is part of the ABI");

bool out_dtype_ok(int32_t dt) { return dt == FB_DT_FLOAT || dt == FB_DT_BFLOAT16 || dt == FB_DT_HALF; }

} // namespace

struct fb_comm {
  fb_device *dev = nullptr;
  int rank = 0, world = 1;
  size_t data_bytes = 0;
  uint8_t *region = nullptr;          // local: header + data (cudaMalloc)
  uint8_t *peer[kMaxRanks] = {nullptr}; // peer[rank] == region
  bool connected = false;
  NcclComm nccl_comm = nullptr;
  NcclId nccl_id;
  bool has_nccl_id = false;
  uint32_t epoch = 0;
  int sm_count = 0;
};

FB_EXPORT fb_status fb_comm_create(fb_device *dev, int32_t rank, int32_t world, size_t buffer_bytes,
                                   fb_comm **out) {
  clear_error();
  FB_REQUIRE(dev && out, FB_INVALID_ARGUMENT, "fb_comm_create: NULL argument");
  *out = nullptr;
  FB_REQUIRE(world >= 1 && world <= kMaxRanks, FB_INVALID_ARGUMENT,
             "fb_comm_create: world size must be 1.." + std::to_string(kMaxRanks));
  FB_REQUIRE(rank >= 0 && rank < world, FB_INVALID_ARGUMENT, "fb_comm_create: rank out of range");
  FB_REQUIRE(buffer_bytes > 0 && buffer_bytes % 256 == 0, FB_INVALID_ARGUMENT,
             "fb_comm_create: buffer size must be a positive multiple of 256 bytes");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  fb_comm *c = new fb_comm();
  c->dev = dev;
  c->rank = rank;
  c->world = world;
  c->data_bytes = buffer_bytes;
  c->sm_count = dev->sm_count;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->region), kHeaderBytes + buffer_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->region, 0, kHeaderBytes);
  if (e != cudaSuccess) {
    if (c->region) cudaFree(c->region);
    delete c;
    return fail(FB_RUNTIME_FAILURE, std::string("fb_comm_create: ") + cudaGetErrorString(e));
  }
  c->peer[rank] = c->region;
  if (world == 1) c->connected = true;
  *out = c;
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_local_handle(fb_comm *comm, uint8_t *block) {
  clear_error();
  FB_REQUIRE(comm && block, FB_INVALID_ARGUMENT, "fb_comm_local_handle: NULL argument");
  IpcBlock b;
  memset(&b, 0, sizeof(b));
  FB_CUDA_OK(cudaSetDevice(comm->dev->ordinal));
  FB_CUDA_OK(cudaIpcGetMemHandle(&b.mem, comm->region));
  b.region_bytes = kHeaderBytes + comm->data_bytes;
  b.rank = (uint32_t)comm->rank;
  if (comm->rank == 0 && comm->world > 1) {
    NcclApi &api = nccl();
    FB_REQUIRE(api.ok, FB_RUNTIME_FAILURE, "fb_comm_local_handle: NCCL unavailable: " + api.why);
    FB_NCCL_OK(api.GetUniqueId(&b.nccl_id));
    b.has_nccl = 1;
  }
  memcpy(block, &b, sizeof(b));
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_connect(fb_comm *comm, const uint8_t *blocks) {
  clear_error();
  FB_REQUIRE(comm && blocks, FB_INVALID_ARGUMENT, "fb_comm_connect: NULL argument");
  FB_REQUIRE(!comm->connected || comm->world == 1, FB_INVALID_ARGUMENT, "fb_comm_connect: already connected");
  if (comm->world == 1) return FB_OK;
  FB_CUDA_OK(cudaSetDevice(comm->dev->ordinal));
  for (int r = 0; r < comm->world; ++r) {
    IpcBlock b;
    memcpy(&b, blocks + (size_t)r * FB_COMM_HANDLE_BYTES, sizeof(b));
    FB_REQUIRE((int)b.rank == r, FB_INVALID_ARGUMENT,
               "fb_comm_connect: block " + std::to_string(r) + " was written by rank " + std::to_string(b.rank));
    FB_REQUIRE(b.region_bytes == kHeaderBytes + comm->data_bytes, FB_INVALID_ARGUMENT,
               "fb_comm_connect: rank " + std::to_string(r) + " created its buffer with a different size");
    if (r == 0) {
      FB_REQUIRE(b.has_nccl == 1, FB_INVALID_ARGUMENT, "fb_comm_connect: rank 0's block carries no NCCL id");
      comm->nccl_id = b.nccl_id;
      comm->has_nccl_id = true;
    }
    if (r == comm->rank) continue;
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, b.mem, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return fail(FB_RUNTIME_FAILURE, "fb_comm_connect: cannot map rank " + std::to_string(r) +
                                          "'s buffer (peer access over NVLink/PCIe is required): " +
                                          cudaGetErrorString(e));
    comm->peer[r] = static_cast<uint8_t *>(p);
  }
  NcclApi &api = nccl();
  FB_REQUIRE(api.ok, FB_RUNTIME_FAILURE, "fb_comm_connect: NCCL unavailable: " + api.why);
  FB_NCCL_OK(api.CommInitRank(&comm->nccl_comm, comm->world, comm->nccl_id, comm->rank));
  comm->connected = true;
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_close(fb_comm *comm) {
  clear_error();
  if (!comm) return FB_OK;
  cudaSetDevice(comm->dev->ordinal);
  cudaStreamSynchronize(comm->dev->stream);
  if (comm->nccl_comm) nccl().CommDestroy(comm->nccl_comm);
  for (int r = 0; r < comm->world; ++r)
    if (r != comm->rank && comm->peer[r]) cudaIpcCloseMemHandle(comm->peer[r]);
  if (comm->region) cudaFree(comm->region);
  delete comm;
  return FB_OK;
}

FB_EXPORT void *fb_comm_buffer(fb_comm *comm) { return comm ? comm->region + kHeaderBytes : nullptr; }
FB_EXPORT size_t fb_comm_buffer_bytes(fb_comm *comm) { return comm ? comm->data_bytes : 0; }
FB_EXPORT int32_t fb_comm_rank(fb_comm *comm) { return comm ? comm->rank : -1; }
FB_EXPORT int32_t fb_comm_world(fb_comm *comm) { return comm ? comm->world : 0; }

static fb_status check_bucket(fb_comm *comm, size_t in_offset, size_t count, size_t out_offset, int32_t out_dtype,
                              const char *who) {
  FB_REQUIRE(comm->connected, FB_INVALID_ARGUMENT, std::string(who) + ": communicator is not connected");
  FB_REQUIRE(out_dtype_ok(out_dtype), FB_INVALID_ARGUMENT, std::string(who) + ": output type must be f32, bf16 or f16");
  FB_REQUIRE(count > 0 && count % 4 == 0, FB_INVALID_ARGUMENT,
             std::string(who) + ": element count must be a positive multiple of 4");
  FB_REQUIRE(in_offset % 16 == 0 && out_offset % 16 == 0, FB_INVALID_ARGUMENT,
             std::string(who) + ": offsets must be multiples of 16 bytes");
  const size_t out_bytes = count * (out_dtype == FB_DT_FLOAT ? 4 : 2);
  FB_REQUIRE(in_offset + count * 4 <= comm->data_bytes && out_offset + out_bytes <= comm->data_bytes,
             FB_INVALID_ARGUMENT, std::string(who) + ": range exceeds the communicator's buffer");
  const bool overlap = in_offset < out_offset + out_bytes && out_offset < in_offset + count * 4;
  FB_REQUIRE(!overlap, FB_INVALID_ARGUMENT, std::string(who) + ": input and output ranges overlap");
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_sum_fused(fb_comm *comm, size_t in_offset, size_t count, size_t out_offset,
                                      int32_t out_dtype) {
  clear_error();
  FB_REQUIRE(comm != nullptr, FB_INVALID_ARGUMENT, "fb_comm_sum_fused: communicator is NULL");
  fb_status st = check_bucket(comm, in_offset, count, out_offset, out_dtype, "fb_comm_sum_fused");
  if (st != FB_OK) return st;
  FB_CUDA_OK(cudaSetDevice(comm->dev->ordinal));
  ExchangeParams p;
  memset(&p, 0, sizeof(p));
  p.world = comm->world;
  p.rank0 = comm->rank;
  p.out_dtype = out_dtype;
  p.epoch = ++comm->epoch;
  p.count = (int64_t)count;
  p.in_off = (int64_t)(kHeaderBytes + in_offset);
  p.out_off = (int64_t)(kHeaderBytes + out_offset);
  for (int r = 0; r < comm->world; ++r) p.region[r] = comm->peer[r];
  p.err = comm->dev->error_word;
  const int64_t vecs_per_rank = ((int64_t)count / 4 + comm->world - 1) / comm->world;
  // All CTAs of the grid wait on peers: never more than one per SM, so they are co-resident.
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(comm->sm_count, (vecs_per_rank + 511) / 512));
  wgrad_exchange_kernel<<<dim3(grid, 1), 512, 0, comm->dev->stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_sum_nccl(fb_comm *comm, void *inout_f32, size_t count, void *out, int32_t out_dtype) {
  clear_error();
  FB_REQUIRE(comm && inout_f32 && out, FB_INVALID_ARGUMENT, "fb_comm_sum_nccl: NULL argument");
  FB_REQUIRE(comm->connected, FB_INVALID_ARGUMENT, "fb_comm_sum_nccl: communicator is not connected");
  FB_REQUIRE(out_dtype_ok(out_dtype), FB_INVALID_ARGUMENT, "fb_comm_sum_nccl: output type must be f32, bf16 or f16");
  FB_REQUIRE(count > 0, FB_INVALID_ARGUMENT, "fb_comm_sum_nccl: empty bucket");
  FB_CUDA_OK(cudaSetDevice(comm->dev->ordinal));
  if (comm->world > 1)
    FB_NCCL_OK(nccl().AllReduce(inout_f32, inout_f32, count, kNcclFloat32, kNcclSum, comm->nccl_comm,
                                comm->dev->stream));
  if (out_dtype == FB_DT_FLOAT) {
    if (out != inout_f32)
      FB_CUDA_OK(cudaMemcpyAsync(out, inout_f32, count * 4, cudaMemcpyDeviceToDevice, comm->dev->stream));
  } else {
    const int blocks = (int)std::min<int64_t>(((int64_t)count + 255) / 256, (int64_t)comm->sm_count * 8);
    cast_f32_kernel<<<blocks, 256, 0, comm->dev->stream>>>(static_cast<const float *>(inout_f32), out, out_dtype,
                                                         (int64_t)count);
    FB_CUDA_OK(cudaGetLastError());
  }
  return FB_OK;
}

FB_EXPORT fb_status fb_comm_allgather(fb_comm *comm, const void *send, void *recv, size_t bytes_per_rank) {
  clear_error();
  FB_REQUIRE(comm && send && recv, FB_INVALID_ARGUMENT, "fb_comm_allgather: NULL argument");
  FB_REQUIRE(comm->connected, FB_INVALID_ARGUMENT, "fb_comm_allgather: communicator is not connected");
  FB_REQUIRE(bytes_per_rank > 0, FB_INVALID_ARGUMENT, "fb_comm_allgather: empty slab");
  FB_CUDA_OK(cudaSetDevice(comm->dev->ordinal));
  if (comm->world == 1) {
    if (send != recv)
      FB_CUDA_OK(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, comm->dev->stream));
    return FB_OK;
  }
  FB_NCCL_OK(nccl().AllGather(send, recv, bytes_per_rank, kNcclInt8, comm->nccl_comm, comm->dev->stream));
  return FB_OK;
}

// Runs the fused exchange for `world` virtual ranks in one cooperative launch on `dev`:
// `buckets` holds world x count fp32 values (rank r's partial at r*count), `out` receives
// world x count values of `out_dtype` (rank r's copy of the sum at r*count). Test entry point.
FB_EXPORT fb_status fb_comm_selftest_emulated(fb_device *dev, int32_t world, const float *buckets, size_t count,
                                              void *out, int32_t out_dtype, int32_t repeats) {
  clear_error();
  FB_REQUIRE(dev && buckets && out, FB_INVALID_ARGUMENT, "fb_comm_selftest_emulated: NULL argument");
  FB_REQUIRE(world >= 1 && world <= kMaxRanks, FB_INVALID_ARGUMENT, "fb_comm_selftest_emulated: bad world size");
  FB_REQUIRE(count > 0 && count % 4 == 0, FB_INVALID_ARGUMENT, "fb_comm_selftest_emulated: count must be a multiple of 4");
  FB_REQUIRE(out_dtype_ok(out_dtype), FB_INVALID_ARGUMENT, "fb_comm_selftest_emulated: bad output type");
  FB_REQUIRE(repeats >= 1, FB_INVALID_ARGUMENT, "fb_comm_selftest_emulated: repeats must be positive");
  FB_CUDA_OK(cudaSetDevice(dev->ordinal));
  const size_t esz = out_dtype == FB_DT_FLOAT ? 4 : 2;
  const size_t in_bytes = (count * 4 + 255) / 256 * 256, out_bytes = (count * esz + 255) / 256 * 256;
  const size_t region_bytes = kHeaderBytes + in_bytes + out_bytes;
  uint8_t *regions = nullptr;
  FB_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&regions), region_bytes * world));
  fb_status st = FB_OK;
  auto body = [&]() -> fb_status {
    FB_CUDA_OK(cudaMemsetAsync(regions, 0, region_bytes * world, dev->stream));
    ExchangeParams p;
    memset(&p, 0, sizeof(p));
    p.world = world;
    p.rank0 = 0;
    p.out_dtype = out_dtype;
    p.count = (int64_t)count;
    p.in_off = (int64_t)kHeaderBytes;
    p.out_off = (int64_t)(kHeaderBytes + in_bytes);
    p.err = dev->error_word;
    for (int r = 0; r < world; ++r) {
      p.region[r] = regions + (size_t)r * region_bytes;
      FB_CUDA_OK(cudaMemcpyAsync(p.region[r] + p.in_off, buckets + (size_t)r * count, count * 4,
                                 cudaMemcpyDeviceToDevice, dev->stream));
    }
    // every virtual rank's CTAs must be resident at once: a cooperative launch checks that
    const int64_t vecs_per_rank = ((int64_t)count / 4 + world - 1) / world;
    int per_rank = (int)std::max<int64_t>(1, std::min<int64_t>(dev->sm_count / world, (vecs_per_rank + 511) / 512));
    for (int it = 0; it < repeats; ++it) {
      p.epoch = (uint32_t)(it + 1);
      void *args[] = {&p};
      FB_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(wgrad_exchange_kernel), dim3(per_rank, world),
                                             dim3(512), args, 0, dev->stream));
    }
    for (int r = 0; r < world; ++r)
      FB_CUDA_OK(cudaMemcpyAsync(static_cast<uint8_t *>(out) + (size_t)r * count * esz, p.region[r] + p.out_off,
                                 count * esz, cudaMemcpyDeviceToDevice, dev->stream));
    FB_CUDA_OK(cudaStreamSynchronize(dev->stream));
    return FB_OK;
  };
  st = body();
  cudaStreamSynchronize(dev->stream);
  cudaFree(regions);
  return st;
}
