#include "devrt.hpp"

#include <cuda.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>

namespace devrt {

namespace {

struct Driver {
  void* lib = nullptr;
  bool ok = false;
  CUresult (*Init)(unsigned) = nullptr;
  CUresult (*DeviceGetCount)(int*) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetName)(char*, int, CUdevice) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DeviceTotalMem)(size_t*, CUdevice) = nullptr;
  CUresult (*DeviceGetPCIBusId)(char*, int, CUdevice) = nullptr;
  CUresult (*DeviceCanAccessPeer)(int*, CUdevice, CUdevice) = nullptr;
  CUresult (*DeviceGetP2PAttribute)(int*, CUdevice_P2PAttribute, CUdevice, CUdevice) = nullptr;
  CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*DevicePrimaryCtxRelease)(CUdevice) = nullptr;
  CUresult (*CtxPushCurrent)(CUcontext) = nullptr;
  CUresult (*CtxPopCurrent)(CUcontext*) = nullptr;
  CUresult (*MemGetInfo)(size_t*, size_t*) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr) = nullptr;
  // optional (symmetric segments): sharing an allocation with other processes through a POSIX file descriptor
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  // optional (multicast object over the blocks of all ranks: one address that NVSwitch fans out to every GPU)
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
};

template <class F>
bool load(void* lib, F& fn, const char* name, const char* fallback = nullptr) {
  void* p = dlsym(lib, name);
  if (!p && fallback) p = dlsym(lib, fallback);
  fn = reinterpret_cast<F>(p);
  return p != nullptr;
}

static bool g_driver_tried = false;

Driver& driver() {
  static Driver d;
  if (g_driver_tried) return d;
  g_driver_tried = true;
  if (d.lib) { dlclose(d.lib); }
  d = Driver{};
  const char* path = std::getenv("B200RT_LIBCUDA");
  d.lib = dlopen(path && path[0] ? path : "libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!d.lib) return d;
  bool ok = true;
  ok &= load(d.lib, d.Init, "cuInit");
  ok &= load(d.lib, d.DeviceGetCount, "cuDeviceGetCount");
  ok &= load(d.lib, d.DeviceGet, "cuDeviceGet");
  ok &= load(d.lib, d.DeviceGetName, "cuDeviceGetName");
  ok &= load(d.lib, d.DeviceGetAttribute, "cuDeviceGetAttribute");
  ok &= load(d.lib, d.DeviceTotalMem, "cuDeviceTotalMem_v2", "cuDeviceTotalMem");
  ok &= load(d.lib, d.DeviceGetPCIBusId, "cuDeviceGetPCIBusId");
  ok &= load(d.lib, d.DeviceCanAccessPeer, "cuDeviceCanAccessPeer");
  ok &= load(d.lib, d.DeviceGetP2PAttribute, "cuDeviceGetP2PAttribute");
  ok &= load(d.lib, d.DevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
  ok &= load(d.lib, d.DevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2", "cuDevicePrimaryCtxRelease");
  ok &= load(d.lib, d.CtxPushCurrent, "cuCtxPushCurrent_v2", "cuCtxPushCurrent");
  ok &= load(d.lib, d.CtxPopCurrent, "cuCtxPopCurrent_v2", "cuCtxPopCurrent");
  ok &= load(d.lib, d.MemGetInfo, "cuMemGetInfo_v2", "cuMemGetInfo");
  ok &= load(d.lib, d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
  ok &= load(d.lib, d.MemAddressReserve, "cuMemAddressReserve");
  ok &= load(d.lib, d.MemAddressFree, "cuMemAddressFree");
  ok &= load(d.lib, d.MemCreate, "cuMemCreate");
  ok &= load(d.lib, d.MemRelease, "cuMemRelease");
  ok &= load(d.lib, d.MemMap, "cuMemMap");
  ok &= load(d.lib, d.MemUnmap, "cuMemUnmap");
  ok &= load(d.lib, d.MemSetAccess, "cuMemSetAccess");
  ok &= load(d.lib, d.PointerGetAttribute, "cuPointerGetAttribute");
  load(d.lib, d.MemExportToShareableHandle, "cuMemExportToShareableHandle");
  load(d.lib, d.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
  load(d.lib, d.MulticastCreate, "cuMulticastCreate");
  load(d.lib, d.MulticastAddDevice, "cuMulticastAddDevice");
  load(d.lib, d.MulticastBindMem, "cuMulticastBindMem");
  load(d.lib, d.MulticastUnbind, "cuMulticastUnbind");
  load(d.lib, d.MulticastGetGranularity, "cuMulticastGetGranularity");
  if (ok && d.Init(0) == CUDA_SUCCESS) d.ok = true;
  return d;
}

int pci_numa_node(const std::string& bus_id) {
  std::string id = bus_id;
  for (auto& c : id) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  const char* root = std::getenv("B200RT_PCI_SYSFS");
  std::ifstream f(std::string(root && root[0] ? root : "/sys/bus/pci/devices") + "/" + id + "/numa_node");
  int n = -1;
  if (f) f >> n;
  return n;
}

struct CtxScope {     // make the device's primary context current for the duration of a call
  Driver& d; CUdevice dev; bool pushed = false;
  CtxScope(Driver& dr, int ordinal) : d(dr), dev(0) {
    CUcontext c = nullptr;
    if (d.DeviceGet(&dev, ordinal) == CUDA_SUCCESS && d.DevicePrimaryCtxRetain(&c, dev) == CUDA_SUCCESS && d.CtxPushCurrent(c) == CUDA_SUCCESS) pushed = true;
  }
  ~CtxScope() { if (pushed) { CUcontext c; d.CtxPopCurrent(&c); d.DevicePrimaryCtxRelease(dev); } }
};

}  // namespace

GpuTopology::GpuTopology() {
  Driver& d = driver();
  if (!d.ok) { status_ = DEVRT_NO_DRIVER; return; }
  int n = 0;
  if (d.DeviceGetCount(&n) != CUDA_SUCCESS) { status_ = DEVRT_NO_DRIVER; return; }
  for (int i = 0; i < n; ++i) {
    GpuInfo g;
    g.ordinal = i;
    CUdevice dev;
    if (d.DeviceGet(&dev, i) != CUDA_SUCCESS) continue;
    char name[256] = {0};
    d.DeviceGetName(name, sizeof name, dev);
    g.name = name;
    d.DeviceGetAttribute(&g.sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dev);
    d.DeviceGetAttribute(&g.cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, dev);
    d.DeviceGetAttribute(&g.cc_minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, dev);
    d.DeviceGetAttribute(&g.multicast_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
    d.DeviceGetAttribute(&g.vmm_supported, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
    d.DeviceTotalMem(&g.mem_total, dev);
    char bus[32] = {0};
    if (d.DeviceGetPCIBusId(bus, sizeof bus, dev) == CUDA_SUCCESS) { g.pci_bus_id = bus; g.numa_node = pci_numa_node(g.pci_bus_id); }
    {
      CtxScope cs(d, i);
      size_t fr = 0, tot = 0;
      if (cs.pushed && d.MemGetInfo(&fr, &tot) == CUDA_SUCCESS) g.mem_free = fr;
    }
    gpus_.push_back(g);
  }
  const int m = num_devices();
  access_.assign(static_cast<size_t>(m) * m, 0);
  atomics_.assign(static_cast<size_t>(m) * m, 0);
  for (int a = 0; a < m; ++a)
    for (int b = 0; b < m; ++b) {
      if (a == b) { access_[a * m + b] = 1; atomics_[a * m + b] = 1; continue; }
      CUdevice da, db;
      d.DeviceGet(&da, a); d.DeviceGet(&db, b);
      int can = 0, at = 0;
      d.DeviceCanAccessPeer(&can, da, db);
      if (can) d.DeviceGetP2PAttribute(&at, CU_DEVICE_P2P_ATTRIBUTE_NATIVE_ATOMIC_SUPPORTED, da, db);
      access_[a * m + b] = can;
      atomics_[a * m + b] = at;
    }
}

int GpuTopology::peer_access(int from, int to) const {
  const int m = num_devices();
  if (from < 0 || to < 0 || from >= m || to >= m) return -1;
  return access_[from * m + to];
}
int GpuTopology::distance(int from, int to) const {
  const int a = peer_access(from, to);
  if (a < 0) return -1;
  if (from == to) return 0;
  if (!a) return -1;
  return atomics_[from * num_devices() + to] ? 1 : 2;
}
DeviceMask GpuTopology::peers_of(int d) const {
  DeviceMask m;
  for (int o = 0; o < num_devices(); ++o) if (o != d && peer_access(d, o) == 1) m.set(o);
  return m;
}
bool GpuTopology::fully_connected() const {
  for (int a = 0; a < num_devices(); ++a)
    for (int b = 0; b < num_devices(); ++b) if (peer_access(a, b) != 1) return false;
  return num_devices() > 0;
}
std::string GpuTopology::debug_string() const {
  std::ostringstream os;
  os << "GPUs: " << num_devices() << (status_ ? " (no driver)" : "") << "\n";
  for (const auto& g : gpus_)
    os << "  gpu " << g.ordinal << ": " << g.name << " sm_" << g.cc_major << g.cc_minor << ", " << g.sm_count << " SMs, "
       << (g.mem_total >> 20) << " MiB total, " << (g.mem_free >> 20) << " MiB free, multicast " << g.multicast_supported
       << ", pci " << g.pci_bus_id << ", numa " << g.numa_node << "\n";
  os << "  peer distance matrix (0 self, 1 NVLink-class, 2 peer w/o atomics, -1 none):\n";
  for (int a = 0; a < num_devices(); ++a) {
    os << "   ";
    for (int b = 0; b < num_devices(); ++b) os << " " << distance(a, b);
    os << "\n";
  }
  return os.str();
}

HbmArena::HbmArena(int device, size_t size, size_t alignment) : alignment_(alignment ? alignment : 1), device_(device) {
  Driver& d = driver();
  if (!d.ok) { status_ = DEVRT_NO_DRIVER; return; }
  if (size == 0 || device < 0) { status_ = DEVRT_BAD_ARG; return; }
  CtxScope cs(d, device);
  if (!cs.pushed) { status_ = DEVRT_BAD_ARG; return; }
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  size_t gran = 0;
  if (d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || gran == 0) { status_ = DEVRT_NO_MEM; return; }
  const size_t bytes = (size + gran - 1) / gran * gran;
  CUdeviceptr va = 0;
  if (d.MemAddressReserve(&va, bytes, 0, 0, 0) != CUDA_SUCCESS) { status_ = DEVRT_NO_MEM; return; }
  CUmemGenericAllocationHandle h = 0;
  if (d.MemCreate(&h, bytes, &prop, 0) != CUDA_SUCCESS) { d.MemAddressFree(va, bytes); status_ = DEVRT_NO_MEM; return; }
  if (d.MemMap(va, bytes, 0, h, 0) != CUDA_SUCCESS) { d.MemRelease(h); d.MemAddressFree(va, bytes); status_ = DEVRT_NO_MEM; return; }
  CUmemAccessDesc acc{};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(va, bytes, &acc, 1) != CUDA_SUCCESS) { d.MemUnmap(va, bytes); d.MemRelease(h); d.MemAddressFree(va, bytes); status_ = DEVRT_NO_MEM; return; }
  base_ = va; handle_ = h; size_ = bytes;
}

HbmArena::~HbmArena() {
  if (!base_) return;
  Driver& d = driver();
  d.MemUnmap(base_, size_);
  d.MemRelease(handle_);
  d.MemAddressFree(base_, size_);
}

uint64_t HbmArena::alloc_bytes(size_t bytes) {
  if (!base_) return 0;
  const size_t start = (offset_ + alignment_ - 1) / alignment_ * alignment_;
  if (start > size_ || bytes > size_ - start) return 0;
  offset_ = start + bytes;
  if (offset_ > high_) high_ = offset_;
  return base_ + start;
}

// ---- SymmSegment -------------------------------------------------------------------------------------------------
SymmSegment::SymmSegment(int device, size_t bytes, int world, int rank) : device_(device), world_(world), rank_(rank) {
  Driver& d = driver();
  if (!d.ok) { status_ = DEVRT_NO_DRIVER; return; }
  if (bytes == 0 || device < 0 || world < 1 || world > 64 || rank < 0 || rank >= world) { status_ = DEVRT_BAD_ARG; return; }
  if (!d.MemExportToShareableHandle || !d.MemImportFromShareableHandle) { status_ = DEVRT_NO_DRIVER; return; }
  CtxScope cs(d, device);
  if (!cs.pushed) { status_ = DEVRT_BAD_ARG; return; }
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) { status_ = DEVRT_NO_MEM; return; }
  // a block that may later be bound to a multicast object has to be a multiple of that object's granularity too
  if (d.MulticastGetGranularity) {
    CUmulticastObjectProp mp{};
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = gran;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (world > 1 && d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran && mg % gran == 0) gran = mg;
  }
  stride_ = (bytes + gran - 1) / gran * gran;
  gran_ = gran;
  CUdeviceptr va = 0;
  if (d.MemAddressReserve(&va, stride_ * world, gran, 0, 0) != CUDA_SUCCESS) { status_ = DEVRT_NO_MEM; return; }
  CUmemGenericAllocationHandle h = 0;
  if (d.MemCreate(&h, stride_, &prop, 0) != CUDA_SUCCESS) { d.MemAddressFree(va, stride_ * world); status_ = DEVRT_NO_MEM; return; }
  base_ = va;
  handles_.assign(world, 0);
  mapped_.assign(world, false);
  handles_[rank] = h;
  if (!map_at(rank, h)) { d.MemRelease(h); d.MemAddressFree(va, stride_ * world); base_ = 0; status_ = DEVRT_NO_MEM; return; }
  int fd = -1;
  if (d.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) { status_ = DEVRT_NO_MEM; fd = -1; }
  fd_ = fd;
}

bool SymmSegment::map_at(int r, uint64_t handle) {
  Driver& d = driver();
  const CUdeviceptr at = base_ + stride_ * static_cast<size_t>(r);
  if (d.MemMap(at, stride_, 0, handle, 0) != CUDA_SUCCESS) return false;
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(at, stride_, &acc, 1) != CUDA_SUCCESS) { d.MemUnmap(at, stride_); return false; }
  mapped_[r] = true;
  return true;
}

int SymmSegment::map_peer(int peer, int fd) {
  Driver& d = driver();
  if (!base_ || peer < 0 || peer >= world_ || peer == rank_ || mapped_[peer] || fd < 0) return DEVRT_BAD_ARG;
  CtxScope cs(d, device_);
  if (!cs.pushed) return DEVRT_BAD_ARG;
  CUmemGenericAllocationHandle h = 0;
  if (d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return DEVRT_NO_MEM;
  if (!map_at(peer, h)) { d.MemRelease(h); return DEVRT_NO_MEM; }
  handles_[peer] = h;
  return 0;
}

int SymmSegment::mc_create() {
  Driver& d = driver();
  if (!base_ || mc_handle_ || !d.MulticastCreate) return DEVRT_NO_DRIVER;
  CtxScope cs(d, device_);
  if (!cs.pushed) return DEVRT_BAD_ARG;
  CUmulticastObjectProp mp{};
  mp.numDevices = static_cast<unsigned>(world_);
  mp.size = stride_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h = 0;
  if (d.MulticastCreate(&h, &mp) != CUDA_SUCCESS) return DEVRT_NO_MEM;
  int fd = -1;
  if (d.MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) { d.MemRelease(h); return DEVRT_NO_MEM; }
  mc_handle_ = h;
  return fd;
}

int SymmSegment::mc_import(int fd) {
  Driver& d = driver();
  if (!base_ || mc_handle_ || fd < 0 || !d.MulticastAddDevice) return DEVRT_BAD_ARG;
  CtxScope cs(d, device_);
  if (!cs.pushed) return DEVRT_BAD_ARG;
  CUmemGenericAllocationHandle h = 0;
  if (d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return DEVRT_NO_MEM;
  mc_handle_ = h;
  return 0;
}

int SymmSegment::mc_add_device() {
  Driver& d = driver();
  if (!mc_handle_ || !d.MulticastAddDevice) return DEVRT_BAD_ARG;
  CtxScope cs(d, device_);
  CUdevice dev;
  if (!cs.pushed || d.DeviceGet(&dev, device_) != CUDA_SUCCESS) return DEVRT_BAD_ARG;
  return d.MulticastAddDevice(mc_handle_, dev) == CUDA_SUCCESS ? 0 : DEVRT_NO_MEM;
}

int SymmSegment::mc_bind() {
  Driver& d = driver();
  if (!mc_handle_ || mc_base_ || !d.MulticastBindMem) return DEVRT_BAD_ARG;
  CtxScope cs(d, device_);
  if (!cs.pushed) return DEVRT_BAD_ARG;
  if (d.MulticastBindMem(mc_handle_, 0, handles_[rank_], 0, stride_, 0) != CUDA_SUCCESS) return DEVRT_NO_MEM;
  mc_bound_ = true;
  CUdeviceptr va = 0;
  if (d.MemAddressReserve(&va, stride_, gran_, 0, 0) != CUDA_SUCCESS) return DEVRT_NO_MEM;
  if (d.MemMap(va, stride_, 0, mc_handle_, 0) != CUDA_SUCCESS) { d.MemAddressFree(va, stride_); return DEVRT_NO_MEM; }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(va, stride_, &acc, 1) != CUDA_SUCCESS) { d.MemUnmap(va, stride_); d.MemAddressFree(va, stride_); return DEVRT_NO_MEM; }
  mc_base_ = va;
  return 0;
}

SymmSegment::~SymmSegment() {
  if (!base_) return;
  Driver& d = driver();
  CtxScope cs(d, device_);
  if (mc_base_) { d.MemUnmap(mc_base_, stride_); d.MemAddressFree(mc_base_, stride_); }
  if (mc_bound_ && d.MulticastUnbind) { CUdevice dev; if (d.DeviceGet(&dev, device_) == CUDA_SUCCESS) d.MulticastUnbind(mc_handle_, dev, 0, stride_); }
  if (mc_handle_) d.MemRelease(mc_handle_);
  for (int r = 0; r < world_; ++r) {
    if (mapped_[r]) d.MemUnmap(base_ + stride_ * static_cast<size_t>(r), stride_);
    if (handles_[r]) d.MemRelease(handles_[r]);
  }
  d.MemAddressFree(base_, stride_ * world_);
}

bool HbmArena::verify_placement() const {
  if (!base_) return false;
  Driver& d = driver();
  int ord = -1;
  if (d.PointerGetAttribute(&ord, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, base_) != CUDA_SUCCESS) return false;
  return ord == device_;
}

}  // namespace devrt

// ---------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------
using namespace devrt;
extern "C" {
// forget the loaded driver so the next call re-reads B200RT_LIBCUDA (tests switch between stand-ins)
void devrt_reload_driver() { g_driver_tried = false; }
void* devrt_topology_create() { return new GpuTopology(); }
void devrt_topology_destroy(void* t) { delete static_cast<GpuTopology*>(t); }
int devrt_topology_status(void* t) { return static_cast<GpuTopology*>(t)->status(); }
int devrt_topology_num_devices(void* t) { return static_cast<GpuTopology*>(t)->num_devices(); }
int devrt_topology_peer_access(void* t, int a, int b) { return static_cast<GpuTopology*>(t)->peer_access(a, b); }
int devrt_topology_distance(void* t, int a, int b) { return static_cast<GpuTopology*>(t)->distance(a, b); }
unsigned long long devrt_topology_peers_of(void* t, int d) { return static_cast<GpuTopology*>(t)->peers_of(d).raw(); }
int devrt_topology_fully_connected(void* t) { return static_cast<GpuTopology*>(t)->fully_connected() ? 1 : 0; }
int devrt_topology_gpu(void* t, int d, char* name, int name_cap, int* sm, int* cc, unsigned long long* total,
                       unsigned long long* free_b, int* multicast, int* numa, char* pci, int pci_cap) {
  const GpuInfo* g = static_cast<GpuTopology*>(t)->gpu(d);
  if (!g) return DEVRT_BAD_ARG;
  std::snprintf(name, name_cap, "%s", g->name.c_str());
  std::snprintf(pci, pci_cap, "%s", g->pci_bus_id.c_str());
  *sm = g->sm_count; *cc = g->cc_major * 10 + g->cc_minor; *total = g->mem_total; *free_b = g->mem_free;
  *multicast = g->multicast_supported; *numa = g->numa_node;
  return 0;
}
int devrt_topology_debug(void* t, char* out, int cap) {
  const std::string s = static_cast<GpuTopology*>(t)->debug_string();
  std::snprintf(out, cap, "%s", s.c_str());
  return static_cast<int>(s.size());
}
void* devrt_arena_create(int device, unsigned long long size, unsigned long long alignment) { return new HbmArena(device, size, alignment); }
void devrt_arena_destroy(void* a) { delete static_cast<HbmArena*>(a); }
int devrt_arena_valid(void* a) { return *static_cast<HbmArena*>(a) ? 1 : 0; }
int devrt_arena_status(void* a) { return static_cast<HbmArena*>(a)->status(); }
unsigned long long devrt_arena_alloc(void* a, unsigned long long bytes) { return static_cast<HbmArena*>(a)->alloc_bytes(bytes); }
unsigned long long devrt_arena_mark(void* a) { return static_cast<HbmArena*>(a)->mark(); }
void devrt_arena_reset_to(void* a, unsigned long long w) { static_cast<HbmArena*>(a)->reset_to(w); }
void devrt_arena_reset(void* a) { static_cast<HbmArena*>(a)->reset(); }
unsigned long long devrt_arena_remaining(void* a) { return static_cast<HbmArena*>(a)->remaining(); }
unsigned long long devrt_arena_used(void* a) { return static_cast<HbmArena*>(a)->used(); }
unsigned long long devrt_arena_size(void* a) { return static_cast<HbmArena*>(a)->size(); }
unsigned long long devrt_arena_high_water(void* a) { return static_cast<HbmArena*>(a)->high_water(); }
unsigned long long devrt_arena_base(void* a) { return static_cast<HbmArena*>(a)->base(); }
int devrt_arena_verify_placement(void* a) { return static_cast<HbmArena*>(a)->verify_placement() ? 1 : 0; }

// symmetric segment: create -> export_fd -> (descriptors cross processes) -> map_peer for every other rank
void* devrt_symm_create(int device, unsigned long long bytes, int world, int rank) {
  auto* s = new (std::nothrow) SymmSegment(device, static_cast<size_t>(bytes), world, rank);
  if (s && !*s) { delete s; return nullptr; }
  return s;
}
void devrt_symm_destroy(void* s) { delete static_cast<SymmSegment*>(s); }
int devrt_symm_export_fd(void* s) { return static_cast<SymmSegment*>(s)->export_fd(); }
int devrt_symm_map_peer(void* s, int peer, int fd) { return static_cast<SymmSegment*>(s)->map_peer(peer, fd); }
unsigned long long devrt_symm_base(void* s) { return static_cast<SymmSegment*>(s)->base(); }
unsigned long long devrt_symm_stride(void* s) { return static_cast<SymmSegment*>(s)->stride(); }
unsigned long long devrt_symm_peer_ptr(void* s, int r) { return static_cast<SymmSegment*>(s)->peer_ptr(r); }
int devrt_symm_mapped(void* s, int r) { return static_cast<SymmSegment*>(s)->mapped(r) ? 1 : 0; }
// multicast object over all ranks' blocks: rank 0 creates (-> descriptor for the others), the others import, everybody
// adds its device, (barrier), everybody binds its block and maps the object, (barrier), mc_ptr() addresses all copies
int devrt_symm_mc_create(void* s) { return static_cast<SymmSegment*>(s)->mc_create(); }
int devrt_symm_mc_import(void* s, int fd) { return static_cast<SymmSegment*>(s)->mc_import(fd); }
int devrt_symm_mc_add_device(void* s) { return static_cast<SymmSegment*>(s)->mc_add_device(); }
int devrt_symm_mc_bind(void* s) { return static_cast<SymmSegment*>(s)->mc_bind(); }
unsigned long long devrt_symm_mc_ptr(void* s) { return static_cast<SymmSegment*>(s)->mc_ptr(); }
}
