// Symmetric memory: one VMM allocation per rank ("segment"), exported as a
// POSIX file descriptor, imported and mapped by every peer, and (when the
// fabric allows it) bound to an NVSwitch multicast object so that one address
// reaches all copies.
//
// Same capability as the reference's ParallelTensor
// (cuMemCreate / cuMemMap / cuMemSetAccess + fd export/import + cuMulticast*:
// datasets/example048_thunderkitten_all_reduce_easy/nv/
// empty_thunderkitten_all_reduce.cu:161-243) and as the cudaIpc hand-off of
// datasets/example012_gpu_ipc_comm_with_NVLink/nv/empty_gpu_ipc_comm.cu:110-180.
// Differences: the world size is a run-time value, one segment backs a whole
// heap (sub-allocated by the Python layer) so a single exchange serves many
// tensors, and every step returns an error code instead of exiting.
//
// The fd exchange itself lives in broker.cc; the Python layer sequences
// create -> export -> exchange -> import -> multicast steps with host barriers.
#include <string.h>
#include <unistd.h>

#include <mutex>
#include <string>
#include <vector>

#include "../prim/status.h"
#include "driver_api.h"

namespace cb {

static thread_local std::string g_last_error;
void set_last_error(const std::string& s) { g_last_error = s; }

const DriverApi& driver_api() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
      api.why = std::string("no CUDA device: ") + cudaGetErrorString(e);
      (void)cudaGetLastError();
      return;
    }
    bool all = true;
    auto get = [&](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      cudaError_t r = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
      if (r != cudaSuccess || q != cudaDriverEntryPointSuccess || *fn == nullptr) {
        all = false;
        api.why += std::string(" missing ") + name;
        (void)cudaGetLastError();
      }
    };
#define CB_GET(n) get(#n, reinterpret_cast<void**>(&api.n))
    CB_GET(cuGetErrorString);
    CB_GET(cuMemCreate);
    CB_GET(cuMemRelease);
    CB_GET(cuMemAddressReserve);
    CB_GET(cuMemAddressFree);
    CB_GET(cuMemMap);
    CB_GET(cuMemUnmap);
    CB_GET(cuMemSetAccess);
    CB_GET(cuMemGetAllocationGranularity);
    CB_GET(cuMemExportToShareableHandle);
    CB_GET(cuMemImportFromShareableHandle);
    CB_GET(cuMulticastCreate);
    CB_GET(cuMulticastAddDevice);
    CB_GET(cuMulticastBindMem);
    CB_GET(cuMulticastUnbind);
    CB_GET(cuMulticastGetGranularity);
    CB_GET(cuDeviceGet);
    CB_GET(cuDeviceGetAttribute);
    CB_GET(cuTensorMapEncodeTiled);
    CB_GET(cuStreamWriteValue32);
#undef CB_GET
    api.ok = all;
  });
  return api;
}

std::string cu_err(const char* what, CUresult r) {
  const char* s = nullptr;
  const DriverApi& d = driver_api();
  if (d.cuGetErrorString) d.cuGetErrorString(r, &s);
  return std::string(what) + " failed: " + (s ? s : "unknown") + " (" + std::to_string(int(r)) +
         ")";
}

struct Segment {
  int device = 0;
  size_t bytes = 0;
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr local = 0;
  CUmemGenericAllocationHandle peer_handle[CB_MAX_RANKS] = {};
  CUdeviceptr peer[CB_MAX_RANKS] = {};
  bool has_mc = false;
  bool mc_bound = false;
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_ptr = 0;
};

static CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

static int set_rw(const DriverApi& d, CUdeviceptr p, size_t bytes, int device) {
  CUmemAccessDesc a;
  memset(&a, 0, sizeof(a));
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUresult r = d.cuMemSetAccess(p, bytes, &a, 1);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemSetAccess", r));
    return -1;
  }
  return 0;
}

}  // namespace cb

using namespace cb;

extern "C" {

const char* cb_last_error() { return g_last_error.c_str(); }

// Stream memory operation: `value` is written to the 4-byte aligned device word `dev_ptr` when
// the stream reaches this point - by the copy engine's front end, without a kernel, so it
// completes even while a persistent kernel occupies every SM.  Used to publish "the rows copied
// so far have landed" to a kernel that is already running.
int cb_stream_write_u32(void* stream, void* dev_ptr, unsigned int value) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error("driver API unavailable:" + d.why);
    return -1;
  }
  CUresult r = d.cuStreamWriteValue32(static_cast<CUstream>(stream),
                                      reinterpret_cast<CUdeviceptr>(dev_ptr), value, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuStreamWriteValue32", r));
    return -1;
  }
  return 0;
}

// 1 when this device supports NVSwitch multicast objects, 0 when not, <0 on error.
int cb_symm_multicast_supported(int device) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error(d.why);
    return -1;
  }
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device) != CUDA_SUCCESS) return -1;
  int v = 0;
  if (d.cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
    return 0;
  return v;
}

// Rounds `bytes` up to what both the allocator and a `world`-device multicast
// object accept, so that every rank computes the same segment size.
long long cb_symm_round_size(int device, long long bytes, int world, int want_mc) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error(d.why);
    return -1;
  }
  CUmemAllocationProp p = local_prop(device);
  size_t g = 0;
  CUresult r = d.cuMemGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemGetAllocationGranularity", r));
    return -1;
  }
  if (want_mc && world > 1) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = size_t(bytes);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
            CUDA_SUCCESS &&
        mg > g)
      g = mg;
  }
  if (g == 0) g = 2u << 20;
  return (long long)(((size_t(bytes) + g - 1) / g) * g);
}

// Allocates and maps the local part of a segment.  `bytes` must come from
// cb_symm_round_size.  Returns an opaque segment pointer in *out.
int cb_symm_segment_create(int device, long long bytes, void** out, void** local_ptr) {
  const DriverApi& d = driver_api();
  if (!d.ok) {
    set_last_error(d.why);
    return -1;
  }
  Segment* s = new Segment();
  s->device = device;
  s->bytes = size_t(bytes);
  CUmemAllocationProp p = local_prop(device);
  CUresult r = d.cuMemCreate(&s->handle, s->bytes, &p, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemCreate", r));
    delete s;
    return -1;
  }
  r = d.cuMemAddressReserve(&s->local, s->bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemAddressReserve", r));
    d.cuMemRelease(s->handle);
    delete s;
    return -1;
  }
  r = d.cuMemMap(s->local, s->bytes, 0, s->handle, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemMap", r));
    d.cuMemAddressFree(s->local, s->bytes);
    d.cuMemRelease(s->handle);
    delete s;
    return -1;
  }
  if (set_rw(d, s->local, s->bytes, device) != 0) {
    d.cuMemUnmap(s->local, s->bytes);
    d.cuMemAddressFree(s->local, s->bytes);
    d.cuMemRelease(s->handle);
    delete s;
    return -1;
  }
  *out = s;
  *local_ptr = reinterpret_cast<void*>(s->local);
  return 0;
}

// POSIX fd for the local allocation; the caller closes it after the exchange.
int cb_symm_segment_export_fd(void* seg) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  int fd = -1;
  CUresult r = d.cuMemExportToShareableHandle(&fd, s->handle,
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemExportToShareableHandle", r));
    return -1;
  }
  return fd;
}

// Maps peer `rank`'s allocation (received as `fd`) into this process.
int cb_symm_segment_import_peer(void* seg, int rank, int fd, void** peer_ptr) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  if (rank < 0 || rank >= CB_MAX_RANKS) {
    set_last_error("peer rank out of range");
    return -1;
  }
  CUmemGenericAllocationHandle h;
  CUresult r = d.cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd,
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemImportFromShareableHandle", r));
    return -1;
  }
  CUdeviceptr p = 0;
  r = d.cuMemAddressReserve(&p, s->bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemAddressReserve(peer)", r));
    d.cuMemRelease(h);
    return -1;
  }
  r = d.cuMemMap(p, s->bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemMap(peer)", r));
    d.cuMemAddressFree(p, s->bytes);
    d.cuMemRelease(h);
    return -1;
  }
  if (set_rw(d, p, s->bytes, s->device) != 0) {
    d.cuMemUnmap(p, s->bytes);
    d.cuMemAddressFree(p, s->bytes);
    d.cuMemRelease(h);
    return -1;
  }
  s->peer_handle[rank] = h;
  s->peer[rank] = p;
  *peer_ptr = reinterpret_cast<void*>(p);
  return 0;
}

// Rank 0 creates the multicast object and gets the fd to broadcast.
int cb_symm_mc_create(void* seg, int world) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = world;
  mp.size = s->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUresult r = d.cuMulticastCreate(&s->mc_handle, &mp);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMulticastCreate", r));
    return -1;
  }
  s->has_mc = true;
  int fd = -1;
  r = d.cuMemExportToShareableHandle(&fd, s->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                     0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemExportToShareableHandle(mc)", r));
    d.cuMemRelease(s->mc_handle);
    s->has_mc = false;
    return -1;
  }
  return fd;
}

int cb_symm_mc_import(void* seg, int fd) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  CUresult r = d.cuMemImportFromShareableHandle(&s->mc_handle, (void*)(uintptr_t)fd,
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemImportFromShareableHandle(mc)", r));
    return -1;
  }
  s->has_mc = true;
  return 0;
}

// Every rank adds its device; a host barrier must follow before anyone binds.
int cb_symm_mc_add_device(void* seg) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  CUdevice dev;
  CUresult r = d.cuDeviceGet(&dev, s->device);
  if (r == CUDA_SUCCESS) r = d.cuMulticastAddDevice(s->mc_handle, dev);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMulticastAddDevice", r));
    return -1;
  }
  return 0;
}

// Binds the local allocation at offset 0 of the object and maps the multicast
// address range.  A host barrier must follow before the address is used.
int cb_symm_mc_bind(void* seg, void** mc_ptr) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  CUresult r = d.cuMulticastBindMem(s->mc_handle, 0, s->handle, 0, s->bytes, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMulticastBindMem", r));
    return -1;
  }
  s->mc_bound = true;
  r = d.cuMemAddressReserve(&s->mc_ptr, s->bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemAddressReserve(mc)", r));
    return -1;
  }
  r = d.cuMemMap(s->mc_ptr, s->bytes, 0, s->mc_handle, 0);
  if (r != CUDA_SUCCESS) {
    set_last_error(cu_err("cuMemMap(mc)", r));
    d.cuMemAddressFree(s->mc_ptr, s->bytes);
    s->mc_ptr = 0;
    return -1;
  }
  if (set_rw(d, s->mc_ptr, s->bytes, s->device) != 0) {
    d.cuMemUnmap(s->mc_ptr, s->bytes);
    d.cuMemAddressFree(s->mc_ptr, s->bytes);
    s->mc_ptr = 0;
    return -1;
  }
  *mc_ptr = reinterpret_cast<void*>(s->mc_ptr);
  return 0;
}

// Unmaps everything.  The caller synchronises the device and runs a host
// barrier first, so that no peer still touches this rank's memory.
int cb_symm_segment_destroy(void* seg) {
  const DriverApi& d = driver_api();
  Segment* s = static_cast<Segment*>(seg);
  if (s == nullptr) return 0;
  if (s->mc_ptr) {
    d.cuMemUnmap(s->mc_ptr, s->bytes);
    d.cuMemAddressFree(s->mc_ptr, s->bytes);
  }
  if (s->has_mc) {
    if (s->mc_bound) {
      CUdevice dev;
      if (d.cuDeviceGet(&dev, s->device) == CUDA_SUCCESS)
        d.cuMulticastUnbind(s->mc_handle, dev, 0, s->bytes);
    }
    d.cuMemRelease(s->mc_handle);
  }
  for (int r = 0; r < CB_MAX_RANKS; ++r) {
    if (s->peer[r]) {
      d.cuMemUnmap(s->peer[r], s->bytes);
      d.cuMemAddressFree(s->peer[r], s->bytes);
      d.cuMemRelease(s->peer_handle[r]);
    }
  }
  if (s->local) {
    d.cuMemUnmap(s->local, s->bytes);
    d.cuMemAddressFree(s->local, s->bytes);
  }
  if (s->handle) d.cuMemRelease(s->handle);
  delete s;
  return 0;
}

// ------------------------------------------------------------ cudaIpc variant
// Fallback when fd export is not permitted: plain device memory shared through
// 64-byte cudaIpc handles (which travel through any byte channel).  No multicast.
int cb_ipc_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, size_t(bytes));
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaMalloc: ") + cudaGetErrorString(e));
    return -1;
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    cudaFree(p);
    return -1;
  }
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}
int cb_ipc_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
int cb_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
int cb_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

// Interprocess event, the second half of the cudaIpc hand-off: the producer
// records it after writing, the consumer makes its stream wait on it.
int cb_ipc_event_create(void** event, unsigned char* handle64) {
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming | cudaEventInterprocess);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaEventCreateWithFlags: ") + cudaGetErrorString(e));
    return -1;
  }
  cudaIpcEventHandle_t h;
  e = cudaIpcGetEventHandle(&h, ev);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaIpcGetEventHandle: ") + cudaGetErrorString(e));
    cudaEventDestroy(ev);
    return -1;
  }
  static_assert(sizeof(h) == 64, "cudaIpcEventHandle_t is 64 bytes");
  memcpy(handle64, &h, 64);
  *event = ev;
  return 0;
}
int cb_ipc_event_open(const unsigned char* handle64, void** event) {
  cudaIpcEventHandle_t h;
  memcpy(&h, handle64, 64);
  cudaEvent_t ev;
  cudaError_t e = cudaIpcOpenEventHandle(&ev, h);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaIpcOpenEventHandle: ") + cudaGetErrorString(e));
    return -1;
  }
  *event = ev;
  return 0;
}
int cb_ipc_event_record(void* event, void* stream) {
  return cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream) == cudaSuccess ? 0 : -1;
}
int cb_ipc_event_wait(void* event, void* stream) {
  return cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0) == cudaSuccess ? 0 : -1;
}
int cb_ipc_event_destroy(void* event) {
  return cudaEventDestroy((cudaEvent_t)event) == cudaSuccess ? 0 : -1;
}

// Host-mapped word(s) the device writes and the host reads without a copy
// (status words, FIFO tails).  Returns host pointer and its device alias.
int cb_mapped_alloc(long long bytes, void** host_ptr, void** dev_ptr) {
  void* h = nullptr;
  cudaError_t e = cudaHostAlloc(&h, size_t(bytes), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaHostAlloc: ") + cudaGetErrorString(e));
    return -1;
  }
  memset(h, 0, size_t(bytes));
  void* dptr = nullptr;
  e = cudaHostGetDevicePointer(&dptr, h, 0);
  if (e != cudaSuccess) {
    set_last_error(std::string("cudaHostGetDevicePointer: ") + cudaGetErrorString(e));
    cudaFreeHost(h);
    return -1;
  }
  *host_ptr = h;
  *dev_ptr = dptr;
  return 0;
}
int cb_mapped_free(void* host_ptr) { return cudaFreeHost(host_ptr) == cudaSuccess ? 0 : -1; }

// Single-process multi-GPU use (one process driving several devices, as the
// reference's P2P examples do): enable peer access both ways between all pairs.
int cb_enable_peer_access_all(int ndev) {
  int cur = 0;
  cudaGetDevice(&cur);
  for (int i = 0; i < ndev; ++i) {
    cudaSetDevice(i);
    for (int j = 0; j < ndev; ++j) {
      if (i == j) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, i, j);
      if (!can) {
        set_last_error("peer access not possible between devices " + std::to_string(i) + " and " +
                       std::to_string(j));
        cudaSetDevice(cur);
        return -1;
      }
      cudaError_t e = cudaDeviceEnablePeerAccess(j, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        set_last_error(std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
        cudaSetDevice(cur);
        return -1;
      }
      (void)cudaGetLastError();
    }
  }
  cudaSetDevice(cur);
  return 0;
}

}  // extern "C"
