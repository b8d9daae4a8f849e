// Tensor-parallel group: NCCL communicator resolved at run time (tp.cu).
#pragma once
#include <nccl.h>
#include <string.h>

#include "common.cuh"

namespace logos {

struct TpGroup {
  int   degree = 1;
  int   rank = 0;
  void* comm = nullptr;  // ncclComm_t
};

logos_status_t tp_unique_id(void* out_128);
logos_status_t tp_init(TpGroup* g, int degree, int rank, const void* unique_id_128);
void tp_destroy(TpGroup* g);
// In-place sum over the group; every rank ends with identical bits.
logos_status_t tp_allreduce_sum_f32(TpGroup* g, float* buf, int64_t count, cudaStream_t st);
logos_status_t tp_allgather_bytes(TpGroup* g, const void* send, void* recv, int64_t bytes_per_rank, cudaStream_t st);

// A block of device memory of the same size on every rank of the group, each rank's block
// mapped into every other rank's address space (CUDA IPC; one process per GPU, one node), for
// kernels that read and write their peers' memory over NVLink directly.
struct TpSymm {
  int    degree = 1, rank = 0;
  size_t bytes = 0;
  void*  base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // base[rank] is this rank's own block
  bool   ok = false;  // false: peers could not be mapped (every rank takes the same decision)
};
// Collective over the group.  On failure to map any peer on any rank, `ok` is false on all
// ranks and nothing stays allocated; the caller falls back to NCCL collectives.
logos_status_t tp_symm_alloc(TpGroup* g, size_t bytes, TpSymm* out, cudaStream_t st);
void tp_symm_free(TpSymm* s);

}  // namespace logos
