// Symmetric memory on the CUDA virtual-memory API, with an NVSwitch multicast mapping on top.
//
// Every rank creates one physical allocation (cuMemCreate, exportable as a POSIX file descriptor),
// maps it into its own address space, hands the descriptor to its peers (the descriptors travel
// over Unix sockets on the Python side) and maps every peer's allocation as well: the same arena
// layout as the CUDA-IPC path (a buffer at offset X is at peer[r] + X on rank r), so every kernel
// of symm_comm.cu runs on it unchanged. Unlike CUDA-IPC memory such an allocation can be bound to a
// multicast object: one more mapping (mc_base) whose loads reduce over all ranks inside the switch
// (multimem.ld_reduce) and whose stores land in every rank's copy (multimem.st).
//
// The reference's symmetric-memory module only names these things
// (tensorplay/distributed/_symmetric_memory/__init__.py:228-432: `multimem_*`, `rendezvous`,
// `get_buffer` are collectives on ordinary tensors); here they are the allocator and the kernels.
#include "sm100.cuh"
#include "tpb_api.h"

#include <string.h>
#include <unistd.h>

namespace tpb {

// ------------------------------------------------------------------ driver entry points
// The library links only the runtime; driver functions are looked up at first use.
struct Drv {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*DeviceGet)(CUdevice*, int);
  bool ok = false;
};

static Drv* drv() {
  static Drv d;
  static bool tried = false;
  if (tried) return d.ok ? &d : nullptr;
  tried = true;
  ensure_thread_context();
  auto get = [](const char* name, void** fn) {
    cudaDriverEntryPointQueryResult q;
    return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess &&
           q == cudaDriverEntryPointSuccess && *fn;
  };
  bool ok = true;
#define TPB_DRV(sym) ok = get("cu" #sym, reinterpret_cast<void**>(&d.sym)) && ok
  TPB_DRV(MemCreate); TPB_DRV(MemRelease); TPB_DRV(MemGetAllocationGranularity);
  TPB_DRV(MemExportToShareableHandle); TPB_DRV(MemImportFromShareableHandle);
  TPB_DRV(MemAddressReserve); TPB_DRV(MemAddressFree); TPB_DRV(MemMap); TPB_DRV(MemUnmap);
  TPB_DRV(MemSetAccess); TPB_DRV(MulticastCreate); TPB_DRV(MulticastAddDevice);
  TPB_DRV(MulticastBindMem); TPB_DRV(MulticastUnbind); TPB_DRV(MulticastGetGranularity);
  TPB_DRV(DeviceGetAttribute); TPB_DRV(DeviceGet);
#undef TPB_DRV
  d.ok = ok;
  return ok ? &d : nullptr;
}

struct VmmState {
  int world = 0, rank = 0, dev = 0;
  size_t bytes = 0;  // size of every rank's allocation (rounded up)
  CUmemGenericAllocationHandle local = 0;
  CUmemGenericAllocationHandle peer_h[16] = {};
  CUdeviceptr va[16] = {};
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false;
};
static VmmState g_vmm;

// symm_comm.cu: installs the mapped arenas as the process's symmetric state.
void symm_adopt(int world, int rank, char* const* peers, size_t bytes, char* mc_base);
void symm_set_mc_base(char* mc_base);

static CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

static int map_handle(Drv* d, CUmemGenericAllocationHandle h, size_t bytes, int dev, CUdeviceptr* out) {
  CUdeviceptr va = 0;
  CUresult r = d->MemAddressReserve(&va, bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  r = d->MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) { d->MemAddressFree(va, bytes); return (int)r; }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d->MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) { d->MemUnmap(va, bytes); d->MemAddressFree(va, bytes); return (int)r; }
  *out = va;
  return 0;
}

}  // namespace tpb

using namespace tpb;

// 1 if this device can export allocations as file descriptors (and `multicast`: join multicast objects).
extern "C" int tpb_symm_vmm_supported(int multicast) {
  Drv* d = drv();
  if (!d) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  CUdevice cd;
  if (d->DeviceGet(&cd, dev) != CUDA_SUCCESS) return 0;
  int v = 0;
  if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd) != CUDA_SUCCESS || !v)
    return 0;
  if (multicast) {
    v = 0;
    if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) != CUDA_SUCCESS || !v) return 0;
  }
  return 1;
}

// Creates this rank's allocation of at least `bytes` (rounded up to the allocation and multicast
// granularities: *bytes_out, identical on every rank for identical requests), zero-filled and
// mapped locally; *fd_out is a descriptor of it for the peers (the caller closes it after sending).
extern "C" int tpb_symm_vmm_create(int world, int rank, size_t bytes, int* fd_out, size_t* bytes_out) {
  Drv* d = drv();
  if (!d) return -5;
  if (world < 1 || world > 16 || rank < 0 || rank >= world) return -2;
  if (g_vmm.local) return -4;
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return (int)ce;
  CUmemAllocationProp prop = alloc_prop(dev);
  size_t gran = 0;
  CUresult r = d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return (int)r;
  if (world > 1 && tpb_symm_vmm_supported(1)) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  const size_t size = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  r = d->MemCreate(&h, size, &prop, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  CUdeviceptr va = 0;
  int rc = map_handle(d, h, size, dev, &va);
  if (rc) { d->MemRelease(h); return rc; }
  ce = cudaMemset(reinterpret_cast<void*>(va), 0, size);
  if (ce != cudaSuccess) return (int)ce;
  int fd = -1;
  r = d->MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  g_vmm = VmmState();
  g_vmm.world = world; g_vmm.rank = rank; g_vmm.dev = dev; g_vmm.bytes = size;
  g_vmm.local = h; g_vmm.va[rank] = va;
  *fd_out = fd;
  *bytes_out = size;
  if (world == 1) {
    char* peers[16] = {};
    peers[0] = reinterpret_cast<char*>(va);
    symm_adopt(1, 0, peers, size, nullptr);
  }
  return 0;
}

// Maps the allocation behind `fd` (received from rank `peer_rank`) into this process. After the last
// peer the arena is complete and becomes the process's symmetric state.
extern "C" int tpb_symm_vmm_map_peer(int peer_rank, int fd) {
  Drv* d = drv();
  if (!d || !g_vmm.local) return -4;
  if (peer_rank < 0 || peer_rank >= g_vmm.world || peer_rank == g_vmm.rank || g_vmm.va[peer_rank]) return -2;
  CUmemGenericAllocationHandle h;
  CUresult r = d->MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return (int)r;
  CUdeviceptr va = 0;
  int rc = map_handle(d, h, g_vmm.bytes, g_vmm.dev, &va);
  if (rc) { d->MemRelease(h); return rc; }
  g_vmm.peer_h[peer_rank] = h;
  g_vmm.va[peer_rank] = va;
  bool all = true;
  for (int i = 0; i < g_vmm.world; ++i) all = all && g_vmm.va[i];
  if (all) {
    char* peers[16] = {};
    for (int i = 0; i < g_vmm.world; ++i) peers[i] = reinterpret_cast<char*>(g_vmm.va[i]);
    symm_adopt(g_vmm.world, g_vmm.rank, peers, g_vmm.bytes, nullptr);
  }
  return 0;
}

// Multicast object over all ranks' allocations. Order (each step on every rank, with a host barrier
// between the steps): rank 0 creates and exports (mc_create), the others import its descriptor
// (mc_import); every rank adds its device (mc_add_device); every rank binds its allocation and
// maps the object (mc_bind).
extern "C" int tpb_symm_mc_create(int* fd_out) {
  Drv* d = drv();
  if (!d || !g_vmm.local) return -4;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = g_vmm.world;
  mp.size = g_vmm.bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUresult r = d->MulticastCreate(&g_vmm.mc, &mp);
  if (r != CUDA_SUCCESS) return (int)r;
  int fd = -1;
  r = d->MemExportToShareableHandle(&fd, g_vmm.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  *fd_out = fd;
  return 0;
}
extern "C" int tpb_symm_mc_import(int fd) {
  Drv* d = drv();
  if (!d || !g_vmm.local) return -4;
  CUresult r = d->MemImportFromShareableHandle(&g_vmm.mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  return (int)r;
}
extern "C" int tpb_symm_mc_add_device() {
  Drv* d = drv();
  if (!d || !g_vmm.mc) return -4;
  CUdevice cd;
  CUresult r = d->DeviceGet(&cd, g_vmm.dev);
  if (r != CUDA_SUCCESS) return (int)r;
  return (int)d->MulticastAddDevice(g_vmm.mc, cd);
}
extern "C" int tpb_symm_mc_bind() {
  Drv* d = drv();
  if (!d || !g_vmm.mc) return -4;
  CUresult r = d->MulticastBindMem(g_vmm.mc, 0, g_vmm.local, 0, g_vmm.bytes, 0);
  if (r != CUDA_SUCCESS) return (int)r;
  g_vmm.mc_bound = true;
  int rc = map_handle(d, g_vmm.mc, g_vmm.bytes, g_vmm.dev, &g_vmm.mc_va);
  if (rc) return rc;
  symm_set_mc_base(reinterpret_cast<char*>(g_vmm.mc_va));
  return 0;
}

// Unmaps and releases everything (call after the last kernel that uses the arena has finished, on
// every rank, with a host barrier before it so that no peer still reads this rank's memory).
extern "C" int tpb_symm_vmm_destroy() {
  Drv* d = drv();
  if (!d || !g_vmm.local) return 0;
  cudaDeviceSynchronize();
  if (g_vmm.mc_va) { d->MemUnmap(g_vmm.mc_va, g_vmm.bytes); d->MemAddressFree(g_vmm.mc_va, g_vmm.bytes); }
  if (g_vmm.mc) {
    if (g_vmm.mc_bound) {
      CUdevice cd;
      if (d->DeviceGet(&cd, g_vmm.dev) == CUDA_SUCCESS) d->MulticastUnbind(g_vmm.mc, cd, 0, g_vmm.bytes);
    }
    d->MemRelease(g_vmm.mc);
  }
  for (int i = 0; i < g_vmm.world; ++i) {
    if (g_vmm.va[i]) { d->MemUnmap(g_vmm.va[i], g_vmm.bytes); d->MemAddressFree(g_vmm.va[i], g_vmm.bytes); }
    if (i != g_vmm.rank && g_vmm.peer_h[i]) d->MemRelease(g_vmm.peer_h[i]);
  }
  d->MemRelease(g_vmm.local);
  g_vmm = VmmState();
  char* none[16] = {};
  symm_adopt(0, 0, none, 0, nullptr);
  return 0;
}
