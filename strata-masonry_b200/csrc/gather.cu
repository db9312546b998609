// The one optional exchange of the column-sharded GEMM behind the C ABI: an NCCL all-gather of the
// [M, N/g] column slabs over NVLink (rank-major [g, M, N/g] on every GPU), followed by the
// library's unshard copy into row-major [M, N].  The reference is single-GPU
// (src/kernels/gemm/sm100a/dense_gemm_bf16.cu:347-348 creates one stream on one device); nothing
// here has a counterpart there.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, preferring a copy the process has
// already loaded), so the library itself has no link-time dependency on it and loads on machines
// without NCCL; the entry points below then return SMB_ERR_UNSUPPORTED.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <new>

#include "gemm_common.cuh"

using namespace smb;

static_assert(sizeof(ncclUniqueId) == SMB_COMM_ID_BYTES, "communicator id size of the C ABI");

namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*);
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  const char* (*GetErrorString)(ncclResult_t);
  bool ok;
};

NcclApi g_nccl = {};
std::once_flag g_nccl_once;

void load_nccl() {
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (h == nullptr) return;
  auto sym = [&](const char* name) { return dlsym(h, name); };
  g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
  g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
  g_nccl.CommInitAll = reinterpret_cast<decltype(g_nccl.CommInitAll)>(sym("ncclCommInitAll"));
  g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
  g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(sym("ncclAllGather"));
  g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(sym("ncclGroupStart"));
  g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(sym("ncclGroupEnd"));
  g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(sym("ncclGetErrorString"));
  g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommInitAll && g_nccl.CommDestroy &&
              g_nccl.AllGather && g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.GetErrorString;
}

const NcclApi* nccl() {
  std::call_once(g_nccl_once, load_nccl);
  return g_nccl.ok ? &g_nccl : nullptr;
}

int nccl_missing() {
  return set_error(SMB_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded: %s", dlerror() ? dlerror() : "not found");
}

int nccl_error(const NcclApi* api, ncclResult_t r, const char* what) {
  return set_error(SMB_ERR_CUDA, "%s: NCCL error %d (%s)", what, static_cast<int>(r), api->GetErrorString(r));
}

}  // namespace

struct smb_comm {
  ncclComm_t comm;
  int world, rank, device;
};

namespace smb {

int comm_world(const smb_comm* comm) { return comm->world; }
int comm_rank(const smb_comm* comm) { return comm->rank; }
int comm_device(const smb_comm* comm) { return comm->device; }

int comm_allgather_inplace(smb_comm* comm, void* buf, size_t block_bytes, cudaStream_t stream) {
  if (comm == nullptr || buf == nullptr) return set_error(SMB_ERR_INVALID, "all-gather: null argument");
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  // NCCL's in-place form: the send buffer is this rank's block inside the receive buffer.
  const char* send = static_cast<const char*>(buf) + static_cast<size_t>(comm->rank) * block_bytes;
  ncclResult_t r = api->AllGather(send, buf, block_bytes, ncclUint8, comm->comm, stream);
  if (r != ncclSuccess) return nccl_error(api, r, "ncclAllGather");
  return SMB_OK;
}

}  // namespace smb

// Shape rules shared by both all-gather entry points; no device needed.
extern "C" int smb_allgather_check(int world, int M, int n_local, int64_t ldd) {
  if (world < 1 || world > 64) return set_error(SMB_ERR_INVALID, "all-gather: world of %d ranks outside 1..64", world);
  if (M <= 0 || n_local <= 0) return set_error(SMB_ERR_INVALID, "all-gather: M and the slab width must be positive");
  if (n_local % 8 != 0)
    return set_error(SMB_ERR_INVALID, "all-gather: slab width %d must be a multiple of 8 (16-byte rows)", n_local);
  if (ldd != 0 && (ldd % 8 != 0 || ldd < static_cast<int64_t>(world) * n_local))
    return set_error(SMB_ERR_INVALID, "all-gather: row pitch %lld of the full D must be a multiple of 8 and >= %lld",
                     static_cast<long long>(ldd), static_cast<long long>(world) * n_local);
  return SMB_OK;
}

extern "C" int smb_comm_unique_id(unsigned char id[SMB_COMM_ID_BYTES]) {
  if (id == nullptr) return set_error(SMB_ERR_INVALID, "communicator id: null output");
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  ncclUniqueId u;
  ncclResult_t r = api->GetUniqueId(&u);
  if (r != ncclSuccess) return nccl_error(api, r, "ncclGetUniqueId");
  std::memcpy(id, &u, sizeof(u));
  return SMB_OK;
}

extern "C" int smb_comm_create(smb_comm** out, const unsigned char id[SMB_COMM_ID_BYTES], int world, int rank) {
  if (out == nullptr || id == nullptr) return set_error(SMB_ERR_INVALID, "communicator: null argument");
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world)
    return set_error(SMB_ERR_INVALID, "communicator: rank %d outside world of %d", rank, world);
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return set_error(SMB_ERR_CUDA, "communicator: no current CUDA device");
  smb_comm* c = new (std::nothrow) smb_comm();
  if (c == nullptr) return set_error(SMB_ERR_NOMEM, "communicator: out of host memory");
  ncclUniqueId u;
  std::memcpy(&u, id, sizeof(u));
  ncclResult_t r = api->CommInitRank(&c->comm, world, u, rank);
  if (r != ncclSuccess) {
    delete c;
    return nccl_error(api, r, "ncclCommInitRank");
  }
  c->world = world;
  c->rank = rank;
  c->device = device;
  *out = c;
  return SMB_OK;
}

extern "C" int smb_comm_create_all(smb_comm** out, int ndev, const int* devices) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "communicators: null output");
  for (int i = 0; i < (ndev > 0 ? ndev : 0); ++i) out[i] = nullptr;
  if (ndev < 1 || ndev > 64) return set_error(SMB_ERR_INVALID, "communicators: %d devices outside 1..64", ndev);
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  ncclComm_t comms[64];
  int devs[64];
  for (int i = 0; i < ndev; ++i) devs[i] = devices != nullptr ? devices[i] : i;
  ncclResult_t r = api->CommInitAll(comms, ndev, devs);
  if (r != ncclSuccess) return nccl_error(api, r, "ncclCommInitAll");
  for (int i = 0; i < ndev; ++i) {
    smb_comm* c = new (std::nothrow) smb_comm();
    if (c == nullptr) {
      for (int j = 0; j < ndev; ++j) {
        if (j < i) delete out[j];
        out[j] = nullptr;
        api->CommDestroy(comms[j]);
      }
      return set_error(SMB_ERR_NOMEM, "communicators: out of host memory");
    }
    c->comm = comms[i];
    c->world = ndev;
    c->rank = i;
    c->device = devs[i];
    out[i] = c;
  }
  return SMB_OK;
}

extern "C" int smb_comm_destroy(smb_comm* comm) {
  if (comm == nullptr) return SMB_OK;
  const NcclApi* api = nccl();
  if (api != nullptr) api->CommDestroy(comm->comm);
  delete comm;
  return SMB_OK;
}

extern "C" int smb_allgather_columns(smb_comm* comm, const void* slab, void* gathered, void* d_full, int M,
                                     int n_local, int64_t ldd, void* stream) {
  if (comm == nullptr) return set_error(SMB_ERR_INVALID, "all-gather: null communicator");
  if (slab == nullptr || gathered == nullptr) return set_error(SMB_ERR_INVALID, "all-gather: null buffer");
  if (int rc = smb_allgather_check(comm->world, M, n_local, d_full != nullptr ? ldd : 0)) return rc;
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device != comm->device)
    return set_error(SMB_ERR_INVALID, "all-gather: communicator of device %d used with device %d current",
                     comm->device, device);
  const size_t count = static_cast<size_t>(M) * n_local;
  ncclResult_t r = api->AllGather(slab, gathered, count, ncclBfloat16, comm->comm, static_cast<cudaStream_t>(stream));
  if (r != ncclSuccess) return nccl_error(api, r, "ncclAllGather");
  if (d_full != nullptr) return smb_unshard_columns_device(gathered, d_full, comm->world, M, n_local, ldd, stream);
  return SMB_OK;
}

extern "C" int smb_allgather_columns_multi(smb_comm* const* comms, int ndev, const void* const* slabs,
                                           void* const* gathered, void* const* d_full, int M, int n_local,
                                           int64_t ldd, void* const* streams) {
  if (comms == nullptr || slabs == nullptr || gathered == nullptr)
    return set_error(SMB_ERR_INVALID, "all-gather: null argument list");
  if (int rc = smb_allgather_check(ndev, M, n_local, d_full != nullptr ? ldd : 0)) return rc;
  for (int i = 0; i < ndev; ++i) {
    if (comms[i] == nullptr || comms[i]->world != ndev || comms[i]->rank != i)
      return set_error(SMB_ERR_INVALID, "all-gather: communicator %d does not belong to this group of %d", i, ndev);
    if (slabs[i] == nullptr || gathered[i] == nullptr || (d_full != nullptr && d_full[i] == nullptr))
      return set_error(SMB_ERR_INVALID, "all-gather: null buffer for device %d", i);
  }
  const NcclApi* api = nccl();
  if (api == nullptr) return nccl_missing();
  int before = 0;
  if (cudaGetDevice(&before) != cudaSuccess) return set_error(SMB_ERR_CUDA, "all-gather: no current CUDA device");
  const size_t count = static_cast<size_t>(M) * n_local;
  // One host thread drives all devices: the calls must sit in one NCCL group.
  ncclResult_t r = api->GroupStart();
  if (r != ncclSuccess) return nccl_error(api, r, "ncclGroupStart");
  ncclResult_t first_bad = ncclSuccess;
  for (int i = 0; i < ndev; ++i) {
    cudaStream_t st = streams != nullptr ? static_cast<cudaStream_t>(streams[i]) : nullptr;
    r = api->AllGather(slabs[i], gathered[i], count, ncclBfloat16, comms[i]->comm, st);
    if (r != ncclSuccess && first_bad == ncclSuccess) first_bad = r;
  }
  r = api->GroupEnd();
  if (first_bad != ncclSuccess) return nccl_error(api, first_bad, "ncclAllGather");
  if (r != ncclSuccess) return nccl_error(api, r, "ncclGroupEnd");
  int rc = SMB_OK;
  if (d_full != nullptr) {
    for (int i = 0; i < ndev && rc == SMB_OK; ++i) {
      cudaError_t e = cudaSetDevice(comms[i]->device);
      if (e != cudaSuccess) {
        rc = set_cuda_error(e, "all-gather: cudaSetDevice");
        break;
      }
      rc = smb_unshard_columns_device(gathered[i], d_full[i], ndev, M, n_local, ldd,
                                      streams != nullptr ? streams[i] : nullptr);
    }
    cudaSetDevice(before);
  }
  return rc;
}
