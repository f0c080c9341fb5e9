// Row- / vocabulary-sharded entry points whose exchange step is an NCCL collective on a
// communicator the host owns: the all-gather of the row shards' outputs and the MAX all-reduce of
// the fused lm_head's (value, index) keys.  These are the only two collectives the path needs.
//
// NCCL is bound at run time (dlopen of libnccl.so.2 on first use), so the library loads on hosts
// without NCCL and a host that already has an NCCL loaded (its own, or a framework's) gets that
// one.  Nothing here creates or destroys communicators: the host passes its ncclComm_t.
#include <dlfcn.h>

#include <mutex>

#include "qmm_common.cuh"

namespace {

// the few NCCL constants the two calls need (nccl.h: ncclDataType_t, ncclRedOp_t)
constexpr int kNcclInt64 = 4, kNcclFloat32 = 7, kNcclMax = 2;

using AllGatherFn = int (*)(const void *, void *, size_t, int, void *, cudaStream_t);
using AllReduceFn = int (*)(const void *, void *, size_t, int, int, void *, cudaStream_t);

std::mutex g_nccl_mutex;
bool g_nccl_tried = false;
AllGatherFn g_all_gather = nullptr;
AllReduceFn g_all_reduce = nullptr;

bool bind_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mutex);
  if (!g_nccl_tried) {
    g_nccl_tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h) {
      g_all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
      g_all_reduce = reinterpret_cast<AllReduceFn>(dlsym(h, "ncclAllReduce"));
    }
  }
  return g_all_gather && g_all_reduce;
}

int nccl_status(int r) { return r == 0 ? COGNI_QMM_OK : COGNI_QMM_ERR_NCCL_BASE + r; }

}  // namespace

extern "C" {

int cogni_qmm_sharded_gemv_nccl(void *nccl_comm, int world, int rank, int type, const void *d_w_shard,
                                const float *d_x, float *d_gather, int in_dim, int rows, int batch,
                                int resident, void *stream) {
  if (!nccl_comm || world < 1 || rank < 0 || rank >= world || !d_gather || rows <= 0 || batch <= 0)
    return COGNI_QMM_ERR_ARG;
  if (!bind_nccl()) return COGNI_QMM_ERR_NCCL_MISSING;
  const size_t count = (size_t)batch * rows;
  float *mine = d_gather + (size_t)rank * count;
  const int st = resident
                     ? cogni_qmm_gemv_resident(type, d_w_shard, d_x, nullptr, 0, mine, in_dim, rows, batch, stream)
                     : cogni_qmm_gemv(type, d_w_shard, d_x, nullptr, 0, mine, in_dim, rows, batch, stream);
  if (st != COGNI_QMM_OK) return st;
  if (world == 1) return COGNI_QMM_OK;
  // in place: rank's block of the receive buffer is the send buffer
  return nccl_status(g_all_gather(mine, d_gather, count, kNcclFloat32, nccl_comm,
                                  static_cast<cudaStream_t>(stream)));
}

int cogni_qmm_sharded_top1_nccl(void *nccl_comm, int world, int type, const void *d_w_shard,
                                const float *d_x, int in_dim, int rows, int batch, int32_t index_base,
                                void *d_scratch, size_t scratch_bytes, int64_t *d_keys,
                                int32_t *d_top_index, float *d_top_value, void *stream) {
  if (!nccl_comm || world < 1 || !d_keys) return COGNI_QMM_ERR_ARG;
  if (!bind_nccl()) return COGNI_QMM_ERR_NCCL_MISSING;
  int st = cogni_qmm_gemv_top1(type, d_w_shard, d_x, in_dim, rows, batch, index_base, d_scratch,
                               scratch_bytes, d_top_index, d_top_value, d_keys, stream);
  if (st != COGNI_QMM_OK || world == 1) return st;
  st = nccl_status(g_all_reduce(d_keys, d_keys, (size_t)batch, kNcclInt64, kNcclMax, nccl_comm,
                                static_cast<cudaStream_t>(stream)));
  if (st != COGNI_QMM_OK) return st;
  return cogni_qmm_top1_unpack_keys(d_keys, batch, d_top_index, d_top_value, stream);
}

}  // extern "C"
