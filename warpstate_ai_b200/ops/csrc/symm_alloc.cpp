// Symmetric memory for the ranks of one node: device allocations that every process maps.
//
// Each rank creates a physical allocation with the CUDA virtual-memory-management API
// (cuMemCreate, POSIX file-descriptor handle type), maps it into its own address space and
// exports it as a file descriptor.  The descriptors travel between the processes over Unix
// sockets (the Python side, parallel/symm.py); a peer imports one and maps it at an address of
// its own.  When the NVSwitch fabric supports it, rank 0 also creates a multicast object of the
// same size, every rank adds its device and binds its allocation, and the object is mapped once
// more: loads from that mapping can reduce across the ranks and stores broadcast (`multimem.*`).
//
// The reference has no such layer (its only collectives are NCCL's through DDP, reference
// run_40b.py:601-603); this is what the in-kernel collectives of comm.cu stand on.
//
// Driver entry points are resolved at run time, so the library does not link against libcuda.
// Nothing here launches a kernel or touches a tensor map; the mappings are plain device memory to
// everything else.  Every function returns 0 or a negative code and, on failure, leaves a text
// for ws_symm_last_error().
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdio.h>
#include <string.h>
#include <string>
#include <unistd.h>

namespace {

struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok = false;
};

thread_local std::string g_error;

int fail(int code, const char* what, CUresult r = CUDA_SUCCESS) {
  char text[256];
  if (r != CUDA_SUCCESS)
    snprintf(text, sizeof(text), "%s (CUresult %d)", what, (int)r);
  else
    snprintf(text, sizeof(text), "%s", what);
  g_error = text;
  return code;
}

template <typename Fn>
bool resolve(const char* name, Fn* out) {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult found;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess ||
      ptr == nullptr)
    return false;
  *out = reinterpret_cast<Fn>(ptr);
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFree(nullptr);  // a current context for the driver calls below
    d.ok = resolve("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity) && resolve("cuMemCreate", &d.MemCreate) &&
           resolve("cuMemExportToShareableHandle", &d.MemExportToShareableHandle) &&
           resolve("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle) &&
           resolve("cuMemAddressReserve", &d.MemAddressReserve) && resolve("cuMemMap", &d.MemMap) &&
           resolve("cuMemSetAccess", &d.MemSetAccess) && resolve("cuMemUnmap", &d.MemUnmap) &&
           resolve("cuMemAddressFree", &d.MemAddressFree) && resolve("cuMemRelease", &d.MemRelease) &&
           resolve("cuMulticastCreate", &d.MulticastCreate) && resolve("cuMulticastAddDevice", &d.MulticastAddDevice) &&
           resolve("cuMulticastBindMem", &d.MulticastBindMem) && resolve("cuMulticastUnbind", &d.MulticastUnbind) &&
           resolve("cuMulticastGetGranularity", &d.MulticastGetGranularity) && resolve("cuDeviceGet", &d.DeviceGet) &&
           resolve("cuDeviceGetAttribute", &d.DeviceGetAttribute);
  });
  return d;
}

CUmemAllocationProp device_memory_on(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// Reserve an address range, map `handle` there and give `device` read/write access.
int map_for_device(Driver& d, CUmemGenericAllocationHandle handle, size_t bytes, size_t alignment, int device,
                   CUdeviceptr* out) {
  CUdeviceptr va = 0;
  CUresult r = d.MemAddressReserve(&va, bytes, alignment, 0, 0);
  if (r != CUDA_SUCCESS) return fail(-42, "cuMemAddressReserve failed", r);
  r = d.MemMap(va, bytes, 0, handle, 0);
  if (r != CUDA_SUCCESS) {
    d.MemAddressFree(va, bytes);
    return fail(-43, "cuMemMap failed", r);
  }
  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(va, bytes, &access, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(va, bytes);
    d.MemAddressFree(va, bytes);
    return fail(-44, "cuMemSetAccess failed", r);
  }
  *out = va;
  return 0;
}

}  // namespace

extern "C" {

const char* ws_symm_last_error(void) { return g_error.c_str(); }

// 1 when `device` can take part in NVSwitch multicast objects, 0 when not, negative on error.
int ws_symm_multicast_supported(int device) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  CUdevice dev;
  int value = 0;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return fail(-41, "cuDeviceGet failed");
  if (d.DeviceGetAttribute(&value, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return value ? 1 : 0;
}

// Size an allocation of `bytes` is rounded up to so that it can be mapped by peers and, for `world` > 1 with
// multicast, bound to a multicast object of the same size.
long long ws_symm_padded_size(int device, long long bytes, int world, int want_multicast) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  if (bytes <= 0) return fail(-41, "size must be positive");
  CUmemAllocationProp prop = device_memory_on(device);
  size_t granule = 0;
  CUresult r = d.MemGetAllocationGranularity(&granule, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || granule == 0) return fail(-41, "cuMemGetAllocationGranularity failed", r);
  if (want_multicast && world > 1) {
    CUmulticastObjectProp mc;
    memset(&mc, 0, sizeof(mc));
    mc.numDevices = static_cast<unsigned>(world);
    mc.size = static_cast<size_t>(bytes);
    mc.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mc_granule = 0;
    if (d.MulticastGetGranularity(&mc_granule, &mc, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mc_granule > granule)
      granule = mc_granule;
  }
  const size_t padded = (static_cast<size_t>(bytes) + granule - 1) / granule * granule;
  return static_cast<long long>(padded);
}

// Create `bytes` (already padded) of device memory on `device`, map it locally and export it.
// handle_out: opaque allocation handle; ptr_out: local device address; fd_out: descriptor to send to peers
// (the caller closes it after sending).
int ws_symm_create(int device, long long bytes, unsigned long long* handle_out, unsigned long long* ptr_out, int* fd_out) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  CUmemAllocationProp prop = device_memory_on(device);
  CUmemGenericAllocationHandle handle;
  CUresult r = d.MemCreate(&handle, static_cast<size_t>(bytes), &prop, 0);
  if (r != CUDA_SUCCESS) return fail(-45, "cuMemCreate failed (out of memory, or the size is not a multiple of the granularity)", r);
  CUdeviceptr va = 0;
  int rc = map_for_device(d, handle, static_cast<size_t>(bytes), 0, device, &va);
  if (rc != 0) {
    d.MemRelease(handle);
    return rc;
  }
  int fd = -1;
  r = d.MemExportToShareableHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(va, static_cast<size_t>(bytes));
    d.MemAddressFree(va, static_cast<size_t>(bytes));
    d.MemRelease(handle);
    return fail(-46, "cuMemExportToShareableHandle failed", r);
  }
  *handle_out = static_cast<unsigned long long>(handle);
  *ptr_out = static_cast<unsigned long long>(va);
  *fd_out = fd;
  return 0;
}

// Map a peer's allocation (received as `fd`) for `device`.  The descriptor stays the caller's to close.
int ws_symm_import(int device, int fd, long long bytes, unsigned long long* handle_out, unsigned long long* ptr_out) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  CUmemGenericAllocationHandle handle;
  CUresult r = d.MemImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return fail(-47, "cuMemImportFromShareableHandle failed", r);
  CUdeviceptr va = 0;
  int rc = map_for_device(d, handle, static_cast<size_t>(bytes), 0, device, &va);
  if (rc != 0) {
    d.MemRelease(handle);
    return rc;
  }
  *handle_out = static_cast<unsigned long long>(handle);
  *ptr_out = static_cast<unsigned long long>(va);
  return 0;
}

// Rank 0: a multicast object for `world` devices of `bytes` each; fd_out goes to every peer.
int ws_symm_multicast_create(long long bytes, int world, unsigned long long* mc_out, int* fd_out) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = static_cast<unsigned>(world);
  prop.size = static_cast<size_t>(bytes);
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc;
  CUresult r = d.MulticastCreate(&mc, &prop);
  if (r != CUDA_SUCCESS) return fail(-48, "cuMulticastCreate failed", r);
  int fd = -1;
  r = d.MemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(mc);
    return fail(-46, "exporting the multicast object failed", r);
  }
  *mc_out = static_cast<unsigned long long>(mc);
  *fd_out = fd;
  return 0;
}

int ws_symm_multicast_import(int fd, unsigned long long* mc_out) {
  Driver& d = driver();
  if (!d.ok) return fail(-40, "the CUDA driver lacks the virtual-memory or multicast entry points");
  CUmemGenericAllocationHandle mc;
  CUresult r = d.MemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return fail(-47, "importing the multicast object failed", r);
  *mc_out = static_cast<unsigned long long>(mc);
  return 0;
}

// Every rank, before any rank binds: add this rank's device to the object.
int ws_symm_multicast_add_device(unsigned long long mc, int device) {
  Driver& d = driver();
  CUdevice dev;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return fail(-41, "cuDeviceGet failed");
  CUresult r = d.MulticastAddDevice(static_cast<CUmemGenericAllocationHandle>(mc), dev);
  return r == CUDA_SUCCESS ? 0 : fail(-49, "cuMulticastAddDevice failed", r);
}

// Every rank, after all devices were added: bind this rank's allocation and map the object.
int ws_symm_multicast_bind(unsigned long long mc, unsigned long long handle, long long bytes, int device,
                           unsigned long long* ptr_out) {
  Driver& d = driver();
  CUresult r = d.MulticastBindMem(static_cast<CUmemGenericAllocationHandle>(mc), 0,
                                  static_cast<CUmemGenericAllocationHandle>(handle), 0, static_cast<size_t>(bytes), 0);
  if (r != CUDA_SUCCESS) return fail(-50, "cuMulticastBindMem failed", r);
  CUdeviceptr va = 0;
  int rc = map_for_device(d, static_cast<CUmemGenericAllocationHandle>(mc), static_cast<size_t>(bytes), 0, device, &va);
  if (rc != 0) {
    CUdevice dev;
    if (d.DeviceGet(&dev, device) == CUDA_SUCCESS)
      d.MulticastUnbind(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0, static_cast<size_t>(bytes));
    return rc;
  }
  *ptr_out = static_cast<unsigned long long>(va);
  return 0;
}

// Undo a multicast mapping of this rank: unmap, unbind this device's memory, drop the object reference.
int ws_symm_multicast_release(unsigned long long mc, unsigned long long mc_ptr, long long bytes, int device, int bound) {
  Driver& d = driver();
  if (mc_ptr != 0) {
    d.MemUnmap(static_cast<CUdeviceptr>(mc_ptr), static_cast<size_t>(bytes));
    d.MemAddressFree(static_cast<CUdeviceptr>(mc_ptr), static_cast<size_t>(bytes));
  }
  if (bound) {
    CUdevice dev;
    if (d.DeviceGet(&dev, device) == CUDA_SUCCESS)
      d.MulticastUnbind(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0, static_cast<size_t>(bytes));
  }
  d.MemRelease(static_cast<CUmemGenericAllocationHandle>(mc));
  return 0;
}

// Undo ws_symm_create / ws_symm_import: unmap the range and drop the allocation reference.
int ws_symm_release(unsigned long long handle, unsigned long long ptr, long long bytes) {
  Driver& d = driver();
  if (ptr != 0) {
    d.MemUnmap(static_cast<CUdeviceptr>(ptr), static_cast<size_t>(bytes));
    d.MemAddressFree(static_cast<CUdeviceptr>(ptr), static_cast<size_t>(bytes));
  }
  d.MemRelease(static_cast<CUmemGenericAllocationHandle>(handle));
  return 0;
}

// A synchronous copy between any two mapped ranges (this GPU's or a peer's) by the driver's copy path --
// no kernel of any library touches the peer mapping.  For tests and one-off transfers.
int ws_symm_copy(unsigned long long dst, unsigned long long src, long long bytes) {
  const cudaError_t e = cudaMemcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src),
                                   static_cast<size_t>(bytes), cudaMemcpyDefault);
  if (e != cudaSuccess) {
    g_error = std::string("cudaMemcpy failed: ") + cudaGetErrorString(e);
    return -48;
  }
  return 0;
}

void ws_symm_close_fd(int fd) {
  if (fd >= 0) close(fd);
}

}  // extern "C"
