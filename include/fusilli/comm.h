// fusilli::Comm -- the multi-GPU exchange of the sharded hot path behind the C ABI's fb_comm_*.
//
// No counterpart in the reference, which has no multi-device code: one Handle is one device
// (reference include/fusilli/backend/handle.h:74-112, `create(backend, deviceId)`). A sharded run
// keeps that unit -- one process (or thread) and one Handle per GPU, one Graph per shard -- and
// adds one Comm per rank for the two things that cross devices: the sum of the fp32 weight-gradient
// partials (fused peer-memory kernel, or NCCL all-reduce + cast) and the gather of output slabs.
//
//   auto comm = Comm::create(handle, rank, world, bytes, allGather);   // collective over the ranks
//   wgradGraph.execute(handle, {{dy, ..}, {x, ..}, {dw, comm.view(off, n * 4)}}, ws);   // fp32 partial
//   comm.sumFused(/*inOffset=*/0, /*count=*/n, /*outOffset=*/outOff, DataType::BFloat16);
//
// `allGather` moves the 256-byte bootstrap blocks between the ranks (MPI, files, a TCP store: any
// function that returns every rank's block in rank order).
#ifndef FUSILLI_COMM_H
#define FUSILLI_COMM_H

#include <functional>
#include <memory>
#include <utility>
#include <vector>

#include "backend.h"

namespace fusilli {

class Comm {
public:
  using Block = std::vector<uint8_t>;
  // Receives this rank's block, returns all ranks' blocks in rank order.
  using AllGather = std::function<ErrorOr<std::vector<Block>>(const Block &)>;

  static ErrorOr<Comm> create(const Handle &handle, int rank, int world, size_t bufferBytes,
                              const AllGather &allGather = {}) {
    bufferBytes = (bufferBytes + 255) / 256 * 256;
    fb_comm *c = nullptr;
    FUSILLI_FB_CALL(fb_comm_create(handle.device(), rank, world, bufferBytes, &c));
    Comm out(c, &handle);
    if (world > 1) {
      FUSILLI_RETURN_ERROR_IF(!allGather, ErrorCode::InvalidArgument, "Comm::create: world > 1 needs an all-gather of bytes");
      Block mine(FB_COMM_HANDLE_BYTES);
      FUSILLI_FB_CALL(fb_comm_local_handle(c, mine.data()));
      FUSILLI_ASSIGN_OR_RETURN(std::vector<Block> all, allGather(mine));
      FUSILLI_RETURN_ERROR_IF(all.size() != static_cast<size_t>(world), ErrorCode::InvalidArgument,
                              "Comm::create: the all-gather returned " + std::to_string(all.size()) + " blocks for " +
                                  std::to_string(world) + " ranks");
      Block flat;
      for (const Block &b : all) {
        FUSILLI_RETURN_ERROR_IF(b.size() != FB_COMM_HANDLE_BYTES, ErrorCode::InvalidArgument,
                                "Comm::create: malformed bootstrap block");
        flat.insert(flat.end(), b.begin(), b.end());
      }
      FUSILLI_FB_CALL(fb_comm_connect(c, flat.data()));
    }
    return ok(std::move(out));
  }

  Comm(const Comm &) = delete;
  Comm &operator=(const Comm &) = delete;
  Comm(Comm &&o) noexcept : comm_(std::exchange(o.comm_, nullptr)), handle_(o.handle_) {}
  Comm &operator=(Comm &&o) noexcept {
    if (this != &o) {
      reset();
      comm_ = std::exchange(o.comm_, nullptr);
      handle_ = o.handle_;
    }
    return *this;
  }
  ~Comm() { reset(); }

  int rank() const { return fb_comm_rank(comm_); }
  int world() const { return fb_comm_world(comm_); }
  size_t bufferBytes() const { return fb_comm_buffer_bytes(comm_); }
  void *bufferPtr() const { return fb_comm_buffer(comm_); }

  // A Buffer over [offset, offset + bytes) of this rank's exchange buffer: bind a weight-gradient
  // output to it or read a summed result from it. The Handle given to create() must be alive.
  ErrorOr<std::shared_ptr<Buffer>> view(size_t offset, size_t bytes) const {
    FUSILLI_RETURN_ERROR_IF(bytes == 0 || offset + bytes > bufferBytes(), ErrorCode::InvalidArgument,
                            "Comm::view: range outside the exchange buffer");
    FUSILLI_ASSIGN_OR_RETURN(Buffer b, Buffer::import(*handle_, static_cast<uint8_t *>(bufferPtr()) + offset, bytes));
    return ok(std::make_shared<Buffer>(std::move(b)));
  }

  ErrorObject sumFused(size_t inOffset, size_t count, size_t outOffset, DataType outType) const {
    return fromStatus(fb_comm_sum_fused(comm_, inOffset, count, outOffset, static_cast<int32_t>(outType)));
  }
  ErrorObject sumNccl(void *inoutF32, size_t count, void *out, DataType outType) const {
    return fromStatus(fb_comm_sum_nccl(comm_, inoutF32, count, out, static_cast<int32_t>(outType)));
  }
  ErrorObject allGather(const void *send, void *recv, size_t bytesPerRank) const {
    return fromStatus(fb_comm_allgather(comm_, send, recv, bytesPerRank));
  }

private:
  Comm(fb_comm *c, const Handle *h) : comm_(c), handle_(h) {}
  void reset() {
    if (comm_) fb_comm_close(comm_);
    comm_ = nullptr;
  }
  fb_comm *comm_ = nullptr;
  const Handle *handle_ = nullptr;
};

} // namespace fusilli

#endif // FUSILLI_COMM_H
