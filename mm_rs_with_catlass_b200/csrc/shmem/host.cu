// Symmetric heap for the GPUs of one box, built on the CUDA virtual-memory-management API.
//
// Every rank (process) creates one physical allocation (cuMemCreate, shareable as a POSIX
// file descriptor), reserves W * heap_bytes of virtual address space and maps rank r's
// allocation at base + r * heap_bytes, so the address of a symmetric object on any peer is
// plain pointer arithmetic inside kernels. File descriptors travel between the local processes
// over abstract unix-domain sockets (SCM_RIGHTS). When the GPUs support NVLS, one multicast
// object spanning all ranks is bound to the same physical memory and mapped as an alias:
// multimem.st / multimem.ld_reduce / multimem.red on that alias act on every rank at once.
//
// This is the counterpart of the external SHMEM library the reference links against
// (shmem_set_attr / shmem_init_attr / shmem_malloc / shmem_free / shmem_finalize,
// examples/00_matmul_allreduce/matmul_allreduce.cpp:239-300). The bump allocator on top of
// the heap lives in Python (parallel/shmem.py): allocation is collective and host-only.
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>
#include <vector>
#include "catcoc/capi.h"
#include "catcoc/host_util.h"

using namespace catcoc::host;

struct CatcocHeap {
  int device = 0, rank = 0, world = 1;
  size_t bytes = 0;              // per-rank heap size (rounded to the allocation granularity)
  CUdeviceptr va = 0;            // base of the W * bytes reservation
  CUmemGenericAllocationHandle handles[CATCOC_MAX_WORLD] = {};
  bool mapped[CATCOC_MAX_WORLD] = {};
  // multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_created = false, mc_added = false, mc_bound = false, mc_mapped = false;
  CUdeviceptr mc_va = 0;
  size_t mc_bytes = 0;
};

namespace {

struct Driver {
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*memAddressFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*memGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*memExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*memImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*multicastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*multicastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*multicastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*multicastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*multicastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*deviceGet)(CUdevice*, int);
  CUresult (*deviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok = false;
};

template <typename T>
bool load(T& fn, const char* name) {
  fn = reinterpret_cast<T>(driver_symbol(name));
  return fn != nullptr;
}

Driver* driver() {
  static Driver d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    bool ok = true;
    ok &= load(d.memCreate, "cuMemCreate");
    ok &= load(d.memRelease, "cuMemRelease");
    ok &= load(d.memAddressReserve, "cuMemAddressReserve");
    ok &= load(d.memAddressFree, "cuMemAddressFree");
    ok &= load(d.memMap, "cuMemMap");
    ok &= load(d.memUnmap, "cuMemUnmap");
    ok &= load(d.memSetAccess, "cuMemSetAccess");
    ok &= load(d.memGetAllocationGranularity, "cuMemGetAllocationGranularity");
    ok &= load(d.memExportToShareableHandle, "cuMemExportToShareableHandle");
    ok &= load(d.memImportFromShareableHandle, "cuMemImportFromShareableHandle");
    ok &= load(d.deviceGet, "cuDeviceGet");
    ok &= load(d.deviceGetAttribute, "cuDeviceGetAttribute");
    // multicast entry points may be missing on old drivers: optional
    load(d.multicastCreate, "cuMulticastCreate");
    load(d.multicastAddDevice, "cuMulticastAddDevice");
    load(d.multicastBindMem, "cuMulticastBindMem");
    load(d.multicastUnbind, "cuMulticastUnbind");
    load(d.multicastGetGranularity, "cuMulticastGetGranularity");
    d.ok = ok;
  }
  return d.ok ? &d : nullptr;
}

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

size_t round_up_sz(size_t a, size_t b) { return (a + b - 1) / b * b; }

int set_access(Driver* d, CUdeviceptr ptr, size_t bytes, int device) {
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CATCOC_CU_OK(d->memSetAccess(ptr, bytes, &acc, 1));
  return 0;
}

}  // namespace

extern "C" int catcoc_heap_multicast_supported(int device) {
  Driver* d = driver();
  if (d == nullptr || d->multicastCreate == nullptr) return 0;
  CUdevice dev;
  if (d->deviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  int v = 0;
  if (d->deviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}

extern "C" int catcoc_heap_create(int device, int rank, int world, int64_t bytes, CatcocHeap** out) {
  if (out == nullptr || world < 1 || world > CATCOC_MAX_WORLD || rank < 0 || rank >= world || bytes <= 0) {
    set_error("heap_create: bad arguments (rank %d world %d bytes %lld)", rank, world, static_cast<long long>(bytes));
    return CATCOC_E_BAD_ARG;
  }
  CATCOC_CUDA_OK(cudaSetDevice(device));
  CATCOC_CUDA_OK(cudaFree(nullptr));  // make sure the primary context exists
  Driver* d = driver();
  if (d == nullptr) return CATCOC_E_DRIVER;

  CUmemAllocationProp prop = alloc_prop(device);
  size_t gran = 0;
  CATCOC_CU_OK(d->memGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (catcoc_heap_multicast_supported(device) && d->multicastGetGranularity != nullptr && world > 1) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = round_up_sz(static_cast<size_t>(bytes), gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d->multicastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran)
      gran = mg;
  }
  CatcocHeap* h = new CatcocHeap();
  h->device = device; h->rank = rank; h->world = world;
  h->bytes = round_up_sz(static_cast<size_t>(bytes), gran);

  CUresult r = d->memCreate(&h->handles[rank], h->bytes, &prop, 0);
  if (r != CUDA_SUCCESS) {
    set_error("cuMemCreate(%zu bytes) failed: CUresult %d", h->bytes, static_cast<int>(r));
    delete h;
    return CATCOC_E_NOMEM;
  }
  r = d->memAddressReserve(&h->va, h->bytes * world, gran, 0, 0);
  if (r != CUDA_SUCCESS) {
    set_error("cuMemAddressReserve failed: CUresult %d", static_cast<int>(r));
    d->memRelease(h->handles[rank]);
    delete h;
    return CATCOC_E_NOMEM;
  }
  r = d->memMap(h->va + h->bytes * rank, h->bytes, 0, h->handles[rank], 0);
  if (r == CUDA_SUCCESS) {
    h->mapped[rank] = true;
    if (set_access(d, h->va + h->bytes * rank, h->bytes, device) != 0) r = CUDA_ERROR_UNKNOWN;
  }
  if (r != CUDA_SUCCESS) {
    set_error("mapping the local heap failed: CUresult %d", static_cast<int>(r));
    catcoc_heap_destroy(h);
    return CATCOC_E_DRIVER;
  }
  CATCOC_CUDA_OK(cudaMemset(reinterpret_cast<void*>(h->va + h->bytes * rank), 0, h->bytes));
  CATCOC_CUDA_OK(cudaDeviceSynchronize());
  *out = h;
  return CATCOC_OK;
}

extern "C" int64_t catcoc_heap_bytes(const CatcocHeap* h) { return h ? static_cast<int64_t>(h->bytes) : 0; }

extern "C" int catcoc_heap_export_fd(CatcocHeap* h) {
  Driver* d = driver();
  if (d == nullptr || h == nullptr) return CATCOC_E_DRIVER;
  int fd = -1;
  CUresult r = d->memExportToShareableHandle(&fd, h->handles[h->rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    set_error("cuMemExportToShareableHandle failed: CUresult %d", static_cast<int>(r));
    return CATCOC_E_DRIVER;
  }
  return fd;
}

extern "C" int catcoc_heap_import_peer(CatcocHeap* h, int peer, int fd) {
  Driver* d = driver();
  if (d == nullptr || h == nullptr) return CATCOC_E_DRIVER;
  if (peer < 0 || peer >= h->world || peer == h->rank || h->mapped[peer]) {
    set_error("heap_import_peer: bad peer %d", peer);
    return CATCOC_E_BAD_ARG;
  }
  CATCOC_CU_OK(d->memImportFromShareableHandle(&h->handles[peer], reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  CUresult r = d->memMap(h->va + h->bytes * peer, h->bytes, 0, h->handles[peer], 0);
  if (r != CUDA_SUCCESS) {
    set_error("cuMemMap of peer %d failed: CUresult %d (heap sizes must match on all ranks)", peer, static_cast<int>(r));
    d->memRelease(h->handles[peer]);
    h->handles[peer] = 0;
    return CATCOC_E_DRIVER;
  }
  h->mapped[peer] = true;
  return set_access(d, h->va + h->bytes * peer, h->bytes, h->device);
}

extern "C" void* catcoc_heap_base(const CatcocHeap* h, int peer) {
  if (h == nullptr || peer < 0 || peer >= h->world || !h->mapped[peer]) return nullptr;
  return reinterpret_cast<void*>(h->va + h->bytes * peer);
}

extern "C" int catcoc_heap_mc_create(CatcocHeap* h) {
  Driver* d = driver();
  if (d == nullptr || h == nullptr || d->multicastCreate == nullptr) { set_error("multicast unavailable"); return CATCOC_E_UNSUPPORTED; }
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned>(h->world);
  mp.size = h->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUresult r = d->multicastCreate(&h->mc_handle, &mp);
  if (r != CUDA_SUCCESS) {
    set_error("cuMulticastCreate failed: CUresult %d", static_cast<int>(r));
    return CATCOC_E_UNSUPPORTED;
  }
  h->mc_created = true;
  int fd = -1;
  r = d->memExportToShareableHandle(&fd, h->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    set_error("export of the multicast handle failed: CUresult %d", static_cast<int>(r));
    return CATCOC_E_DRIVER;
  }
  return fd;
}

extern "C" int catcoc_heap_mc_join(CatcocHeap* h, int fd) {
  Driver* d = driver();
  if (d == nullptr || h == nullptr || d->multicastAddDevice == nullptr) { set_error("multicast unavailable"); return CATCOC_E_UNSUPPORTED; }
  if (fd >= 0) {
    CATCOC_CU_OK(d->memImportFromShareableHandle(&h->mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    h->mc_created = true;
  }
  if (!h->mc_created) { set_error("mc_join before mc_create/import"); return CATCOC_E_BAD_ARG; }
  CUdevice dev;
  CATCOC_CU_OK(d->deviceGet(&dev, h->device));
  CATCOC_CU_OK(d->multicastAddDevice(h->mc_handle, dev));
  h->mc_added = true;
  return CATCOC_OK;
}

extern "C" int catcoc_heap_mc_bind(CatcocHeap* h) {
  Driver* d = driver();
  if (d == nullptr || h == nullptr || !h->mc_added) { set_error("mc_bind before mc_join"); return CATCOC_E_BAD_ARG; }
  CATCOC_CU_OK(d->multicastBindMem(h->mc_handle, 0, h->handles[h->rank], 0, h->bytes, 0));
  h->mc_bound = true;
  h->mc_bytes = h->bytes;
  CATCOC_CU_OK(d->memAddressReserve(&h->mc_va, h->mc_bytes, 0, 0, 0));
  CUresult r = d->memMap(h->mc_va, h->mc_bytes, 0, h->mc_handle, 0);
  if (r != CUDA_SUCCESS) {
    set_error("mapping the multicast object failed: CUresult %d", static_cast<int>(r));
    return CATCOC_E_DRIVER;
  }
  h->mc_mapped = true;
  return set_access(d, h->mc_va, h->mc_bytes, h->device);
}

extern "C" void* catcoc_heap_mc_base(const CatcocHeap* h) {
  return (h != nullptr && h->mc_mapped) ? reinterpret_cast<void*>(h->mc_va) : nullptr;
}

// Idempotent teardown in dependency order: multicast mapping -> binding -> handle, then the
// peer mappings, the reservation and the physical handles. The caller must make sure (host
// barrier) that no rank still runs kernels that touch this heap.
extern "C" int catcoc_heap_destroy(CatcocHeap* h) {
  if (h == nullptr) return CATCOC_OK;
  Driver* d = driver();
  if (d == nullptr) { delete h; return CATCOC_E_DRIVER; }
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  if (h->mc_mapped) { d->memUnmap(h->mc_va, h->mc_bytes); h->mc_mapped = false; }
  if (h->mc_va) { d->memAddressFree(h->mc_va, h->mc_bytes); h->mc_va = 0; }
  if (h->mc_bound && d->multicastUnbind != nullptr) {
    CUdevice dev;
    if (d->deviceGet(&dev, h->device) == CUDA_SUCCESS) d->multicastUnbind(h->mc_handle, dev, 0, h->mc_bytes);
    h->mc_bound = false;
  }
  if (h->mc_created) { d->memRelease(h->mc_handle); h->mc_created = false; }
  for (int r = 0; r < h->world; ++r) {
    if (h->mapped[r]) { d->memUnmap(h->va + h->bytes * r, h->bytes); h->mapped[r] = false; }
    if (h->handles[r]) { d->memRelease(h->handles[r]); h->handles[r] = 0; }
  }
  if (h->va) { d->memAddressFree(h->va, h->bytes * h->world); h->va = 0; }
  delete h;
  return CATCOC_OK;
}

// ---------------------------------------------------------------------------------------
// File-descriptor passing between local processes (abstract unix socket, SCM_RIGHTS)
// ---------------------------------------------------------------------------------------
static socklen_t abstract_addr(const char* name, sockaddr_un* addr) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  size_t n = strlen(name);
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  addr->sun_path[0] = '\0';  // abstract namespace: no filesystem entry, vanishes with the socket
  memcpy(addr->sun_path + 1, name, n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

extern "C" int catcoc_fd_recv_open(const char* sock_name) {
  int s = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (s < 0) { set_error("socket(): %s", strerror(errno)); return CATCOC_E_IO; }
  sockaddr_un addr;
  socklen_t len = abstract_addr(sock_name, &addr);
  if (bind(s, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    set_error("bind(%s): %s", sock_name, strerror(errno));
    close(s);
    return CATCOC_E_IO;
  }
  return s;
}

extern "C" int catcoc_fd_recv(int listen_sock, int timeout_ms, int* tag) {
  pollfd pfd = {listen_sock, POLLIN, 0};
  int pr = poll(&pfd, 1, timeout_ms);
  if (pr <= 0) { set_error("fd_recv: timed out after %d ms waiting for a peer", timeout_ms); return CATCOC_E_IO; }
  char data = 0;
  iovec iov = {&data, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov; msg.msg_iovlen = 1;
  msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(listen_sock, &msg, 0) < 0) { set_error("recvmsg: %s", strerror(errno)); return CATCOC_E_IO; }
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
    set_error("fd_recv: message carried no file descriptor");
    return CATCOC_E_IO;
  }
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  if (tag != nullptr) *tag = static_cast<unsigned char>(data);
  return fd;
}

extern "C" int catcoc_fd_send(const char* sock_name, int fd, int tag, int timeout_ms) {
  int s = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (s < 0) { set_error("socket(): %s", strerror(errno)); return CATCOC_E_IO; }
  sockaddr_un addr;
  socklen_t len = abstract_addr(sock_name, &addr);
  char data = static_cast<char>(tag);
  iovec iov = {&data, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_name = &addr; msg.msg_namelen = len;
  msg.msg_iov = &iov; msg.msg_iovlen = 1;
  msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  // the receiver may not have bound its socket yet: retry until the time budget ends
  int waited = 0;
  while (true) {
    if (sendmsg(s, &msg, 0) >= 0) break;
    if ((errno != ECONNREFUSED && errno != ENOENT) || waited >= timeout_ms) {
      set_error("sendmsg(%s): %s", sock_name, strerror(errno));
      close(s);
      return CATCOC_E_IO;
    }
    usleep(2000);
    waited += 2;
  }
  close(s);
  return CATCOC_OK;
}

extern "C" int catcoc_fd_close(int fd) { return close(fd) == 0 ? CATCOC_OK : CATCOC_E_IO; }
