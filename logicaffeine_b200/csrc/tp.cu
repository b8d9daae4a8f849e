// Tensor-parallel plumbing: an NCCL communicator per model, loaded at run time.
//
// The library does not link NCCL: the first tensor-parallel model resolves
// libnccl.so.2 with dlopen (the copy the host process already loaded, e.g.
// the one bundled with PyTorch, wins by soname), so single-GPU users carry no
// NCCL dependency.  Only sum all-reduce (partial o_proj / down_proj outputs when the
// exchange is not folded into the norm kernel) and all-gather (the ranks' CUDA-IPC
// handles at set-up) are used.
#include "tp.cuh"

#include <dlfcn.h>

#include <mutex>

namespace logos {

namespace {
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.handle) break;
    }
    if (!a.handle) return;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(a.handle, "ncclAllGather"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.AllGather && a.GetErrorString;
  });
  return a;
}

logos_status_t nccl_fail(ncclResult_t r, const char* what) {
  return fail(LOGOS_ERROR, "NCCL error %d (%s) in %s", (int)r, api().GetErrorString ? api().GetErrorString(r) : "?", what);
}
}  // namespace

logos_status_t tp_unique_id(void* out_128) {
  NcclApi& a = api();
  if (!a.ok) return fail(LOGOS_ERROR, "tensor parallelism needs libnccl.so.2, which could not be loaded");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = a.GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(out_128, &id, 128);
  return LOGOS_OK;
}

logos_status_t tp_init(TpGroup* g, int degree, int rank, const void* unique_id_128) {
  g->degree = degree;
  g->rank = rank;
  g->comm = nullptr;
  if (degree <= 1) return LOGOS_OK;
  NcclApi& a = api();
  if (!a.ok) return fail(LOGOS_ERROR, "tensor parallelism needs libnccl.so.2, which could not be loaded");
  if (!unique_id_128) return fail(LOGOS_NULL_POINTER, "tp_degree > 1 needs the group's NCCL unique id");
  ncclUniqueId id;
  memcpy(&id, unique_id_128, 128);
  ncclComm_t comm = nullptr;
  ncclResult_t r = a.CommInitRank(&comm, degree, id, rank);
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
  g->comm = comm;
  return LOGOS_OK;
}

void tp_destroy(TpGroup* g) {
  if (g->comm && api().ok) api().CommDestroy(reinterpret_cast<ncclComm_t>(g->comm));
  g->comm = nullptr;
}

logos_status_t tp_allreduce_sum_f32(TpGroup* g, float* buf, int64_t count, cudaStream_t st) {
  if (g->degree <= 1) return LOGOS_OK;
  ncclResult_t r = api().AllReduce(buf, buf, (size_t)count, ncclFloat32, ncclSum, reinterpret_cast<ncclComm_t>(g->comm), st);
  if (r != ncclSuccess) return nccl_fail(r, "ncclAllReduce");
  return LOGOS_OK;
}

logos_status_t tp_allgather_bytes(TpGroup* g, const void* send, void* recv, int64_t bytes_per_rank, cudaStream_t st) {
  if (g->degree <= 1) return LOGOS_OK;
  ncclResult_t r = api().AllGather(send, recv, (size_t)bytes_per_rank, ncclInt8, reinterpret_cast<ncclComm_t>(g->comm), st);
  if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather");
  return LOGOS_OK;
}

logos_status_t tp_symm_alloc(TpGroup* g, size_t bytes, TpSymm* out, cudaStream_t st) {
  *out = TpSymm();
  out->degree = g->degree;
  out->rank = g->rank;
  out->bytes = bytes;
  if (g->degree <= 1 || g->degree > 8) return LOGOS_OK;
  void* local = nullptr;
  LOGOS_CUDA_TRY(cudaMalloc(&local, bytes));
  LOGOS_CUDA_TRY(cudaMemset(local, 0, bytes));
  cudaIpcMemHandle_t mine;
  bool good = cudaIpcGetMemHandle(&mine, local) == cudaSuccess;
  if (!good) cudaGetLastError();
  // exchange the handles (and each rank's outcome so far) through the group's own all-gather
  struct Slot { cudaIpcMemHandle_t h; int32_t good; int32_t pad[15]; };
  static_assert(sizeof(Slot) == 128, "exchange slot");
  Slot send_h;
  memset(&send_h, 0, sizeof(send_h));
  send_h.h = mine;
  send_h.good = good ? 1 : 0;
  Slot* dev = nullptr;
  LOGOS_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&dev), sizeof(Slot) * (size_t)(g->degree + 1)));
  LOGOS_CUDA_TRY(cudaMemcpyAsync(dev + g->degree, &send_h, sizeof(Slot), cudaMemcpyHostToDevice, st));
  logos_status_t rc = tp_allgather_bytes(g, dev + g->degree, dev, (int64_t)sizeof(Slot), st);
  Slot all[8];
  if (rc == LOGOS_OK) {
    LOGOS_CUDA_TRY(cudaMemcpyAsync(all, dev, sizeof(Slot) * (size_t)g->degree, cudaMemcpyDeviceToHost, st));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(st));
  }
  if (rc != LOGOS_OK) {
    cudaFree(dev);
    cudaFree(local);
    return rc;
  }
  for (int r = 0; r < g->degree; ++r) good = good && all[r].good == 1;
  out->base[g->rank] = local;
  if (good) {
    for (int r = 0; r < g->degree && good; ++r) {
      if (r == g->rank) continue;
      void* p = nullptr;
      if (cudaIpcOpenMemHandle(&p, all[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        good = false;
      } else {
        out->base[r] = p;
      }
    }
  }
  // second round: did every rank map every peer?
  send_h.good = good ? 1 : 0;
  LOGOS_CUDA_TRY(cudaMemcpyAsync(dev + g->degree, &send_h, sizeof(Slot), cudaMemcpyHostToDevice, st));
  rc = tp_allgather_bytes(g, dev + g->degree, dev, (int64_t)sizeof(Slot), st);
  if (rc == LOGOS_OK) {
    LOGOS_CUDA_TRY(cudaMemcpyAsync(all, dev, sizeof(Slot) * (size_t)g->degree, cudaMemcpyDeviceToHost, st));
    LOGOS_CUDA_TRY(cudaStreamSynchronize(st));
    for (int r = 0; r < g->degree; ++r) good = good && all[r].good == 1;
  } else {
    good = false;
  }
  cudaFree(dev);
  out->ok = good;
  if (!good) tp_symm_free(out);
  return rc;
}

void tp_symm_free(TpSymm* s) {
  for (int r = 0; r < 8; ++r) {
    if (!s->base[r]) continue;
    if (r == s->rank) cudaFree(s->base[r]);
    else cudaIpcCloseMemHandle(s->base[r]);
    s->base[r] = nullptr;
  }
  s->ok = false;
}

}  // namespace logos

extern "C" logos_status_t logos_tp_unique_id(void* out_128_bytes) {
  return logos::guarded([&]() -> logos_status_t {
    if (!out_128_bytes) return logos::fail(LOGOS_NULL_POINTER, "logos_tp_unique_id: out is null");
    return logos::tp_unique_id(out_128_bytes);
  });
}
