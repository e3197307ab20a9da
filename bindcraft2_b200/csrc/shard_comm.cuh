// Exchange steps of the axially sharded Evoformer stack (one long complex split over P GPUs: rank r holds the band of
// N/P pair rows starting at r*N/P; the reference runs one complex on one GPU, bindcraft/af/native.py:906-975, so this
// has no counterpart there).
//
// Three collectives are all the sharded stack needs: an all-to-all of equal chunks (row band <-> channel group of the
// triangle-multiplication planes, row band <-> column band of the pair stream), an all-gather (attention pair bias,
// outer-product cotangent) and a float sum (attention bias gradient).  Two carriers:
//   NcclComm   one process per GPU; NCCL is bound at run time (dlopen of libnccl.so.2: the library keeps no link-time
//              dependency on it and still loads where NCCL is absent); the unique id travels through the host
//              framework's own process group.
//   LocalComm  P ranks as P host threads of ONE process on ONE GPU, for tests on a single device: exchanges are
//              device-to-device copies between the ranks' buffers behind host barriers.  No kernel ever waits on
//              another kernel; only host threads wait, after synchronising their own stream.
#pragma once
#include <dlfcn.h>
#include <nccl.h>

#include <condition_variable>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "weights.cuh"

namespace bc2 {

struct ShardComm {
  int P = 1, rank = 0;
  virtual ~ShardComm() {}
  // recv[r*bytes, (r+1)*bytes) <- bytes [me*bytes, (me+1)*bytes) of rank r's send buffer
  virtual void all_to_all(const void* send, void* recv, size_t bytes, cudaStream_t st) = 0;
  // recv[r*bytes, (r+1)*bytes) <- rank r's send buffer; send may be recv + rank*bytes (in place)
  virtual void all_gather(const void* send, void* recv, size_t bytes, cudaStream_t st) = 0;
  // buf <- sum over ranks of buf
  virtual void all_reduce_f32(float* buf, size_t count, cudaStream_t st) = 0;
};

// ------------------------------------------------------------------------------------------- NCCL, bound at run time
struct NcclApi {
  void* h = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;

  static NcclApi& get() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
      // RTLD_NOLOAD first: a host framework that already carries NCCL (torch) decides which copy is used
      void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
      api.h = h;
      if (!h) return;
      auto sym = [&](const char* n) { return dlsym(h, n); };
      api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
      api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
      api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
      api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
      api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
      api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
      api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
      api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
      api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
      api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    });
    BC2_CHECK(api.h && api.GetUniqueId && api.CommInitRank && api.GroupStart && api.GroupEnd && api.Send && api.Recv &&
                  api.AllGather && api.AllReduce,
              "NCCL (libnccl.so.2) could not be loaded: the sharded stack needs it for more than one process");
    return api;
  }
};

#define BC2_NCCL(expr)                                                                                       \
  do {                                                                                                       \
    ncclResult_t r_ = (expr);                                                                                \
    if (r_ != ncclSuccess) {                                                                                 \
      NcclApi& a_ = NcclApi::get();                                                                          \
      throw Error(std::string("NCCL: ") + (a_.GetErrorString ? a_.GetErrorString(r_) : "error") + " in " #expr); \
    }                                                                                                        \
  } while (0)

struct NcclComm : ShardComm {
  ncclComm_t comm = nullptr;
  NcclComm(int world, int rank_, const ncclUniqueId& id) {
    P = world;
    rank = rank_;
    BC2_NCCL(NcclApi::get().CommInitRank(&comm, world, id, rank_));
  }
  ~NcclComm() override {
    if (comm && NcclApi::get().CommDestroy) NcclApi::get().CommDestroy(comm);
  }
  void all_to_all(const void* send, void* recv, size_t bytes, cudaStream_t st) override {
    NcclApi& n = NcclApi::get();
    // this rank's own chunk never leaves the device: a plain copy instead of a send/receive pair with itself
    BC2_CUDA(cudaMemcpyAsync(static_cast<char*>(recv) + (size_t)rank * bytes, static_cast<const char*>(send) + (size_t)rank * bytes,
                             bytes, cudaMemcpyDeviceToDevice, st));
    if (P == 1) return;
    BC2_NCCL(n.GroupStart());
    for (int r = 0; r < P; ++r) {
      if (r == rank) continue;
      BC2_NCCL(n.Send(static_cast<const char*>(send) + (size_t)r * bytes, bytes, ncclChar, r, comm, st));
      BC2_NCCL(n.Recv(static_cast<char*>(recv) + (size_t)r * bytes, bytes, ncclChar, r, comm, st));
    }
    BC2_NCCL(n.GroupEnd());
  }
  void all_gather(const void* send, void* recv, size_t bytes, cudaStream_t st) override {
    BC2_NCCL(NcclApi::get().AllGather(send, recv, bytes, ncclChar, comm, st));
  }
  void all_reduce_f32(float* buf, size_t count, cudaStream_t st) override {
    BC2_NCCL(NcclApi::get().AllReduce(buf, buf, count, ncclFloat, ncclSum, comm, st));
  }
};

// ------------------------------------------------------------------------------------------- ranks as host threads
constexpr int kMaxLocalRanks = 8;

struct PeerPtrs {
  const float* p[kMaxLocalRanks];
};
// out = sum of the first P arrays, added in rank order (every rank gets the same bits)
__global__ void sum_peers_kernel(PeerPtrs in, int P, float* __restrict__ out, size_t count) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  float s = in.p[0][i];
  for (int r = 1; r < P; ++r) s += in.p[r][i];
  out[i] = s;
}

// State shared by the P rank threads.  `issue` serialises everything the threads do between two exchanges (kernel
// launches, plan set-up), so the rest of the library needs no thread-safety beyond what it has: a rank thread holds it
// except while it waits in a barrier.
struct LocalWorld {
  int P = 1;
  std::mutex issue;
  std::mutex m;
  std::condition_variable cv;
  int waiting = 0;
  long generation = 0;
  bool failed = false;
  const void* pub[kMaxLocalRanks] = {nullptr};
  explicit LocalWorld(int p) : P(p) { BC2_CHECK(p >= 1 && p <= kMaxLocalRanks, "1 to 8 local ranks"); }
  void fail() {
    std::lock_guard<std::mutex> l(m);
    failed = true;
    cv.notify_all();
  }
  // called with `issue` held through `held`; releases it while waiting
  void barrier(std::unique_lock<std::mutex>& held) {
    held.unlock();
    {
      std::unique_lock<std::mutex> l(m);
      const long g = generation;
      if (++waiting == P) {
        waiting = 0;
        ++generation;
        cv.notify_all();
      } else {
        cv.wait(l, [&] { return generation != g || failed; });
      }
    }
    held.lock();
    if (failed) throw Error("another local rank failed");
  }
};

struct LocalComm : ShardComm {
  LocalWorld* w = nullptr;
  std::unique_lock<std::mutex>* held = nullptr;  // the rank thread's hold on w->issue
  float* tmp = nullptr;                          // all_reduce result before it replaces the operand
  size_t tmp_count = 0;
  DeviceArena* arena = nullptr;
  LocalComm(LocalWorld* w_, int rank_, DeviceArena* a) : w(w_), arena(a) {
    P = w_->P;
    rank = rank_;
  }
  // publish my pointer, meet the others (their streams are drained: what they published is complete)
  void meet(const void* mine, cudaStream_t st) {
    BC2_CUDA(cudaStreamSynchronize(st));
    w->pub[rank] = mine;
    w->barrier(*held);
  }
  // my copies are done; nobody may reuse a published buffer before everybody is here
  void part(cudaStream_t st) {
    BC2_CUDA(cudaStreamSynchronize(st));
    w->barrier(*held);
  }
  void all_to_all(const void* send, void* recv, size_t bytes, cudaStream_t st) override {
    meet(send, st);
    for (int r = 0; r < P; ++r)
      BC2_CUDA(cudaMemcpyAsync(static_cast<char*>(recv) + (size_t)r * bytes,
                               static_cast<const char*>(w->pub[r]) + (size_t)rank * bytes, bytes, cudaMemcpyDeviceToDevice, st));
    part(st);
  }
  void all_gather(const void* send, void* recv, size_t bytes, cudaStream_t st) override {
    meet(send, st);
    for (int r = 0; r < P; ++r) {
      char* dst = static_cast<char*>(recv) + (size_t)r * bytes;
      if (dst == w->pub[r]) continue;  // in place: my own band is already there
      BC2_CUDA(cudaMemcpyAsync(dst, w->pub[r], bytes, cudaMemcpyDeviceToDevice, st));
    }
    part(st);
  }
  void all_reduce_f32(float* buf, size_t count, cudaStream_t st) override {
    if (tmp_count < count) {
      tmp = arena->alloc<float>(count);
      tmp_count = count;
    }
    meet(buf, st);
    PeerPtrs pp{};
    for (int r = 0; r < P; ++r) pp.p[r] = static_cast<const float*>(w->pub[r]);
    launch_counter()++;
    sum_peers_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(pp, P, tmp, count);
    part(st);
    BC2_CUDA(cudaMemcpyAsync(buf, tmp, count * 4, cudaMemcpyDeviceToDevice, st));
  }
};

}  // namespace bc2
