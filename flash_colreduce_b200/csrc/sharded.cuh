// Multi-GPU entry points: one process (rank) per GPU.  Host-only logic plus two
// small kernels; included by colreduce_sm100.cu after run_colreduce.
//
// The reference has no multi-GPU path.  Heads are independent and so are the
// query rows of a head (the softmax normalises per row, flash_colreduce/
// naive.py:19-37), so a rank that holds a subset of the rows of a head produces
// a partial N-vector per head that is combined with + (sum, mean) or max across
// the ranks; the mean divisor of flash_colreduce/flash.py:377-384 is applied
// after the combination.  The one collective is an all-reduce over NCCL, which
// is loaded at run time (dlopen of libnccl.so.2: the copy already in the
// process, e.g. the one PyTorch brought, else the system's), so the library
// itself has no link-time dependency on it.
#pragma once
#include <dlfcn.h>

namespace fcr {

// ------------------------------------------------------------------- shard plan
// Same rule as flash_colreduce_b200.sharding.plan_shards: with at least as many heads as
// ranks the heads are partitioned; otherwise world / heads ranks share a head, its rows are cut
// into 2 * ranks_per_head chunks of whole 128-row tiles and rank g of the head takes chunks g and
// 2 * ranks_per_head - 1 - g (zig-zag: with a causal mask the work of a row grows with its index).
inline int plan_shards_host(int heads, int M, int world, int rank, fcr_shard& s, std::string& err) {
  memset(&s, 0, sizeof(s));
  if (heads <= 0 || M <= 0 || world <= 0 || rank < 0 || rank >= world) {
    err = "fcr_plan_shards: heads, M, world must be positive and 0 <= rank < world";
    return FCR_ERR_BAD_ARG;
  }
  s.rank = rank;
  s.world = world;
  if (heads >= world) {
    const int base = heads / world, extra = heads % world;
    s.head_lo = rank * base + std::min(rank, extra);
    s.head_hi = s.head_lo + base + (rank < extra ? 1 : 0);
    s.n_ranges = 1;
    s.row_lo[0] = 0;
    s.row_hi[0] = M;
    return FCR_OK;
  }
  const int per_head = world / heads;  // ranks that share one head; leftover ranks stay idle
  const int head = rank / per_head, g = rank % per_head;
  s.needs_reduce = 1;
  if (head >= heads) return FCR_OK;  // idle rank: no heads, takes part in the all-reduce only
  s.head_lo = head;
  s.head_hi = head + 1;
  if (per_head == 1) {
    s.n_ranges = 1;
    s.row_lo[0] = 0;
    s.row_hi[0] = M;
    return FCR_OK;
  }
  const int chunks = 2 * per_head;
  long long step = ((long long)M + chunks - 1) / chunks;
  step = (step + kTile - 1) / kTile * kTile;
  const int pick[2] = {g, chunks - 1 - g};
  for (int c : pick) {
    const long long lo = std::min<long long>(c * step, M), hi = std::min<long long>((c + 1) * step, M);
    if (hi > lo) {
      s.row_lo[s.n_ranges] = (int)lo;
      s.row_hi[s.n_ranges] = (int)hi;
      ++s.n_ranges;
    }
  }
  return FCR_OK;
}

// ------------------------------------------------------------------------ NCCL
// The handful of NCCL entry points used, resolved once.
struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(void*) = nullptr;
  int (*CommInitRank)(void**, int, /* ncclUniqueId by value: 128 bytes */ struct NcclId, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string error;
};
struct NcclId {
  char bytes[FCR_NCCL_ID_BYTES];
};
constexpr int kNcclFloat32 = 7;  // ncclFloat32 of nccl.h
constexpr int kNcclSum = 0, kNcclMax = 2;

static NcclApi& nccl_api() {
  static NcclApi api = []() {
    NcclApi a;
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) {
      a.error = std::string("libnccl.so.2 could not be loaded: ") + dlerror();
      return a;
    }
    auto sym = [&](const char* name) {
      void* f = dlsym(a.handle, name);
      if (!f && a.error.empty()) a.error = std::string("libnccl.so.2 has no symbol ") + name;
      return f;
    };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    return a;
  }();
  return api;
}
static int nccl_fail(int rc, const char* what) {
  NcclApi& a = nccl_api();
  return fail(FCR_ERR_NCCL, std::string(what) + ": " + (a.GetErrorString ? a.GetErrorString(rc) : "NCCL error") +
                                " (" + std::to_string(rc) + ")");
}

// ---------------------------------------------------------------------- kernels
// acc[head0 + h][j] (op)= part[h][j] for j < n_part; rows of acc are n_acc long.
__global__ void fold_partial_kernel(float* __restrict__ acc, const float* __restrict__ part, int heads,
                                    int n_part, int n_acc, int head0, int is_max) {
  const size_t total = (size_t)heads * n_part;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t h = idx / n_part, j = idx - h * n_part;
    float* dst = acc + (head0 + h) * (size_t)n_acc + j;
    *dst = is_max ? fmaxf(*dst, part[idx]) : *dst + part[idx];
  }
}

// The row slice [lo, hi) of this rank's heads as a problem of its own: row i of the slice
// attends keys j <= i + c + lo, keys beyond the last row's reach are left out.
static fcr_problem slice_problem(const fcr_problem& local, int lo, int hi) {
  fcr_problem p = local;
  const int64_t c = local.N > local.M ? (int64_t)local.N - local.M : 0;
  p.M = hi - lo;
  if (local.is_causal) {
    p.N = (int32_t)std::min<int64_t>(local.N, c + hi);
    p.causal_offset = c + lo;
  } else {
    p.causal_offset = -1;
  }
  p.reduction = local.reduction == FCR_MAX ? FCR_MAX : FCR_SUM;  // the mean divisor comes last
  p.mean_M = p.mean_N = 0;
  return p;
}

static int sharded_layout(const fcr_problem& local, const fcr_shard& sh, const DeviceInfo& dev, int64_t* off_part,
                          int64_t* total) {
  int64_t need = 0;
  for (int r = 0; r < sh.n_ranges; ++r) {
    const fcr_problem p = slice_problem(local, sh.row_lo[r], sh.row_hi[r]);
    std::string err;
    fcr_plan pl;
    const int rc = plan_problem(p, dev.sms, pl, err);
    if (rc != FCR_OK) return fail(rc, err);
    need = std::max<int64_t>(need, pl.workspace_bytes);
  }
  need = align_up64(need, 256);
  *off_part = need;
  *total = need + align_up64((int64_t)local.B * local.H * local.N * 4, 256);
  return FCR_OK;
}

static int check_shard(const fcr_problem* local, const fcr_shard* sh) {
  if (!local || !sh) return fail(FCR_ERR_BAD_ARG, "null problem or shard");
  if (sh->n_ranges < 0 || sh->n_ranges > 2 || sh->head_hi < sh->head_lo)
    return fail(FCR_ERR_BAD_ARG, "malformed shard");
  if (sh->head_hi - sh->head_lo != local->B * local->H && sh->head_hi > sh->head_lo)
    return fail(FCR_ERR_BAD_ARG, "the local problem must hold exactly the shard's heads (B * H = head_hi - head_lo)");
  for (int r = 0; r < sh->n_ranges; ++r)
    if (sh->row_lo[r] < 0 || sh->row_hi[r] <= sh->row_lo[r] || sh->row_hi[r] > local->M)
      return fail(FCR_ERR_BAD_ARG, "row range outside [0, M)");
  return FCR_OK;
}

}  // namespace fcr

using namespace fcr;

extern "C" {

int fcr_plan_shards(int32_t heads, int32_t M, int32_t world, int32_t rank, fcr_shard* out) {
  if (!out) return fail(FCR_ERR_BAD_ARG, "null shard");
  std::string err;
  const int rc = plan_shards_host(heads, M, world, rank, *out, err);
  return rc == FCR_OK ? rc : fail(rc, err);
}

int fcr_comm_unique_id(void* id_out) {
  if (!id_out) return fail(FCR_ERR_BAD_ARG, "null id");
  NcclApi& a = nccl_api();
  if (!a.error.empty()) return fail(FCR_ERR_NCCL, a.error);
  const int rc = a.GetUniqueId(id_out);
  return rc == 0 ? FCR_OK : nccl_fail(rc, "ncclGetUniqueId");
}

int fcr_comm_init(const void* id, int32_t world, int32_t rank, void** comm_out) {
  if (!id || !comm_out || world <= 0 || rank < 0 || rank >= world)
    return fail(FCR_ERR_BAD_ARG, "null id / comm or rank outside [0, world)");
  NcclApi& a = nccl_api();
  if (!a.error.empty()) return fail(FCR_ERR_NCCL, a.error);
  NcclId nid;
  memcpy(nid.bytes, id, sizeof(nid.bytes));
  void* comm = nullptr;
  const int rc = a.CommInitRank(&comm, world, nid, rank);
  if (rc != 0) return nccl_fail(rc, "ncclCommInitRank");
  *comm_out = comm;
  return FCR_OK;
}

int fcr_comm_destroy(void* comm) {
  if (!comm) return FCR_OK;
  NcclApi& a = nccl_api();
  if (!a.error.empty()) return fail(FCR_ERR_NCCL, a.error);
  const int rc = a.CommDestroy(comm);
  return rc == 0 ? FCR_OK : nccl_fail(rc, "ncclCommDestroy");
}

size_t fcr_sharded_workspace_bytes(const fcr_problem* local, const fcr_shard* shard) {
  if (check_shard(local, shard) != FCR_OK) return 0;
  if (shard->head_hi == shard->head_lo) return 256;
  const DeviceInfo* dev = nullptr;
  if (device_info(&dev, false) != FCR_OK) return 0;
  int64_t off_part = 0, total = 0;
  if (sharded_layout(*local, *shard, *dev, &off_part, &total) != FCR_OK) return 0;
  return (size_t)total;
}

int fcr_colreduce_sharded(const fcr_problem* local, const fcr_shard* shard, int32_t total_heads, const void* q,
                          const void* k, float* acc, void* out, int32_t out_dtype, void* workspace,
                          size_t workspace_bytes, void* comm, void* stream_v) {
  int rc = check_shard(local, shard);
  if (rc != FCR_OK) return rc;
  if (!acc || !out || total_heads <= 0 || shard->head_hi > total_heads)
    return fail(FCR_ERR_BAD_ARG, "null acc / out or head range beyond total_heads");
  if (out_dtype != FCR_F16 && out_dtype != FCR_BF16 && out_dtype != FCR_F32)
    return fail(FCR_ERR_BAD_ARG, "invalid out_dtype");
  if (shard->world > 1 && !comm) return fail(FCR_ERR_BAD_ARG, "a communicator is needed when world > 1");
  const int heads = shard->head_hi - shard->head_lo;
  if (heads > 0 && (!q || !k)) return fail(FCR_ERR_BAD_ARG, "null q or k");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const DeviceInfo* dev = nullptr;
  rc = device_info(&dev, true);
  if (rc != FCR_OK) return rc;
  rc = check_mailbox(*dev, nullptr);
  if (rc != FCR_OK) return rc;
  const fcr_problem& lp = *local;
  const int N = lp.N;
  const bool is_max = lp.reduction == FCR_MAX;
  // zeros are neutral for both operators: partial sums add, probabilities are >= 0
  cudaError_t e = cudaMemsetAsync(acc, 0, (size_t)total_heads * N * sizeof(float), stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(acc)");
  if (heads > 0) {
    int64_t off_part = 0, total = 0;
    rc = sharded_layout(lp, *shard, *dev, &off_part, &total);
    if (rc != FCR_OK) return rc;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || (int64_t)workspace_bytes < total)
      return fail(FCR_ERR_WORKSPACE, "workspace missing, misaligned or smaller than fcr_sharded_workspace_bytes() = " +
                                         std::to_string(total));
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    float* part = reinterpret_cast<float*>(ws + off_part);
    const size_t elem = lp.in_dtype == FCR_F32 ? 4 : 2;
    for (int r = 0; r < shard->n_ranges; ++r) {
      const fcr_problem sp = slice_problem(lp, shard->row_lo[r], shard->row_hi[r]);
      const fcr_plan* pl = nullptr;
      rc = plan_for_call(sp, *dev, &pl);
      if (rc != FCR_OK) return rc;
      const uint8_t* q_rows = reinterpret_cast<const uint8_t*>(q) + (size_t)shard->row_lo[r] * lp.q_strides[2] * elem;
      rc = run_colreduce(sp, *pl, *dev, q_rows, k, part, FCR_F32, ws, (size_t)off_part, stream);
      if (rc != FCR_OK) return rc;
      const size_t n_el = (size_t)heads * sp.N;
      const int blocks = (int)std::min<size_t>((n_el + 255) / 256, 4096);
      g_launches.fetch_add(1, std::memory_order_relaxed);
      fold_partial_kernel<<<blocks, 256, 0, stream>>>(acc, part, heads, sp.N, N, shard->head_lo, is_max ? 1 : 0);
      e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "fold_partial launch");
    }
  }
  if (shard->world > 1) {
    NcclApi& a = nccl_api();
    if (!a.error.empty()) return fail(FCR_ERR_NCCL, a.error);
    const int nrc = a.AllReduce(acc, acc, (size_t)total_heads * N, kNcclFloat32, is_max ? kNcclMax : kNcclSum, comm, stream);
    if (nrc != 0) return nccl_fail(nrc, "ncclAllReduce");
  }
  return fcr_finalize(acc, out, out_dtype, 1, total_heads, lp.M, N, lp.reduction, lp.is_causal, stream_v);
}

}  // extern "C"
