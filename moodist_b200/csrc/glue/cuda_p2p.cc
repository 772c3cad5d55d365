#include "cuda_p2p.h"

#include <c10/cuda/CUDAGuard.h>

#include "core/cuda_group.h"
#include "core/log.h"
#include "core/symm_heap.h"
#include "core/wire.h"
#include "kernels/kernels_api.h"

namespace moodist {
namespace {

constexpr int kFlagWords = 1024;

void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) fail(std::string("moodist: ") + what + " failed: " + cudaGetErrorString(e));
}

struct Ack {
  HostGroup* host;
  int src_rank;
  uint32_t buf_id;
};

// Runs on a driver thread once the receiver's stream has finished the copy; no CUDA calls allowed here.
void CUDART_CB ack_callback(void* p) {
  Ack* a = static_cast<Ack*>(p);
  try {
    a->host->send_message(a->src_rank, kOpCudaItemDone, encode(a->buf_id));
  } catch (...) {
  }
  delete a;
}

}  // namespace

CudaP2P::CudaP2P(CudaGroup& group, HostGroup& host, int device)
    : group_(group), host_(host), heap_(SymmHeap::instance(device)), device_(device) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  flags_ = static_cast<uint32_t*>(heap_.alloc(kFlagWords * sizeof(uint32_t)));
  if (!flags_) fail("moodist: no symmetric memory left for the point-to-point flag words");
  // zeroed on a stream of its own: nothing here may wait for work the caller has queued on its streams
  cudaStream_t s = nullptr;
  cuda_check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
  cuda_check(cudaMemsetAsync(flags_, 0, kFlagWords * sizeof(uint32_t), s), "cudaMemsetAsync");
  cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  cudaStreamDestroy(s);
  host_.set_handler(kOpCudaItemDone, [this](int, Reader& r) { release(r.read<uint32_t>()); });
}

CudaP2P::~CudaP2P() {
  host_.set_handler(kOpCudaItemDone, nullptr);
  std::lock_guard<std::mutex> lk(mu_);
  for (auto& [id, h] : held_)
    if (h.staged) heap_.free(h.staged);
  held_.clear();
  if (flags_) heap_.free(flags_);
}

size_t CudaP2P::held() const {
  std::lock_guard<std::mutex> lk(mu_);
  return held_.size();
}

void CudaP2P::release(uint32_t buf_id) {
  Held gone;
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = held_.find(buf_id);
    if (it == held_.end()) return;
    if (--it->second.remaining > 0) return;
    gone = std::move(it->second);
    held_.erase(it);
  }
  if (gone.staged) heap_.free(gone.staged);  // host-side bookkeeping only: fine on the engine thread
}

void CudaP2P::drop(const CudaItemDescriptor& d) {
  if (d.magic != kCudaItemMagic) return;
  Held gone;
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = held_.find(d.buf_id);
    if (it == held_.end()) return;
    gone = std::move(it->second);
    held_.erase(it);
  }
  if (gone.staged) heap_.free(gone.staged);
}

CudaItemDescriptor CudaP2P::publish(const at::Tensor& t, int readers, cudaStream_t stream) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_);
  const size_t bytes = (size_t)t.nbytes();
  CudaItemDescriptor d;
  d.magic = kCudaItemMagic;
  d.src_rank = group_.rank();
  d.bytes = bytes;
  Held h;
  h.remaining = readers;
  const uint8_t* src = static_cast<const uint8_t*>(t.data_ptr());
  int64_t off = bytes ? heap_.offset_of(src, bytes) : 0;
  if (bytes && off < 0) {
    h.staged = heap_.alloc(bytes);
    if (!h.staged) fail("moodist: no symmetric memory left to stage a CUDA tensor for its receiver");
    cuda_check(cudaMemcpyAsync(h.staged, src, bytes, cudaMemcpyDeviceToDevice, stream), "cudaMemcpyAsync");
    off = heap_.offset_of(h.staged, bytes);
  } else {
    h.keep = t;  // peers read the tensor in place: it must stay alive until they are done
  }
  d.heap_off = (uint64_t)off;
  uint32_t slot;
  {
    std::lock_guard<std::mutex> lk(mu_);
    d.buf_id = ++next_buf_;
    d.flag_val = ++next_flag_val_;
    slot = d.flag_val % kFlagWords;
    held_[d.buf_id] = std::move(h);
  }
  d.flag_off = (uint64_t)heap_.offset_of(flags_ + slot, sizeof(uint32_t));
  // values only grow, so a receiver that still waits for an older value of a reused word is released as well
  if (mb_flag_set(flags_ + slot, d.flag_val, stream) != MB_OK) fail("moodist: could not launch the flag kernel");
  return d;
}

void CudaP2P::fetch(const CudaItemDescriptor& d, void* dst, cudaStream_t stream) {
  if (d.magic != kCudaItemMagic) fail("moodist: not a CUDA item descriptor");
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_);
  const mb_comm_t* comm = static_cast<const mb_comm_t*>(group_.comm_struct());
  if (d.src_rank < 0 || d.src_rank >= comm->world) fail("moodist: CUDA item from an unknown rank");
  const uint8_t* base = static_cast<const uint8_t*>(d.src_rank == comm->rank ? heap_.base() : comm->peer[d.src_rank]);
  if (!base) fail("moodist: the sender's memory is not mapped here");
  group_.check_status();
  if (mb_flag_wait(reinterpret_cast<const uint32_t*>(base + d.flag_off), d.flag_val, comm->status, comm->wait_ns,
                   0x205u | ((uint32_t)d.src_rank << 16), stream) != MB_OK)
    fail("moodist: could not launch the flag kernel");
  if (d.bytes)
    cuda_check(cudaMemcpyAsync(dst, base + d.heap_off, d.bytes, cudaMemcpyDeviceToDevice, stream), "cudaMemcpyAsync");
  Ack* a = new Ack{&host_, d.src_rank, d.buf_id};
  cudaError_t e = cudaLaunchHostFunc(stream, ack_callback, a);
  if (e != cudaSuccess) {
    delete a;
    cuda_check(e, "cudaLaunchHostFunc");
  }
}

}  // namespace moodist
