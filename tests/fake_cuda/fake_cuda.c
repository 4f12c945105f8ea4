/* Host-memory stand-in for the handful of CUDA driver entry points the device runtime uses, so that topology and
 * arena logic can be tested on a machine without a GPU.  FAKE_CUDA_DEVICES (default 2) sets the device count,
 * FAKE_CUDA_NO_PEER=1 removes peer access, FAKE_CUDA_FAIL_CREATE=1 makes physical allocation fail. */
#define _GNU_SOURCE
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

typedef int CUresult;
typedef int CUdevice;
typedef void* CUcontext;
typedef unsigned long long CUdeviceptr;
typedef unsigned long long CUmemGenericAllocationHandle;

static int ndev(void) { const char* e = getenv("FAKE_CUDA_DEVICES"); return e ? atoi(e) : 2; }
static int flag(const char* n) { const char* e = getenv(n); return e && e[0] == '1'; }

typedef struct { unsigned long long va; size_t size; int device; } Mapping;
static Mapping maps[64];
static int nmaps = 0;
static int cur_dev = 0;

CUresult cuInit(unsigned f) { (void)f; return 0; }
CUresult cuDeviceGetCount(int* n) { *n = ndev(); return 0; }
CUresult cuDeviceGet(CUdevice* d, int o) { if (o < 0 || o >= ndev()) return 101; *d = o; return 0; }
CUresult cuDeviceGetName(char* name, int len, CUdevice d) { snprintf(name, len, "Fake B200 #%d", d); return 0; }
CUresult cuDeviceGetAttribute(int* v, int attr, CUdevice d) {
  (void)d;
  switch (attr) {
    case 16: *v = 148; break;        /* MULTIPROCESSOR_COUNT */
    case 75: *v = 10; break;         /* COMPUTE_CAPABILITY_MAJOR */
    case 76: *v = 0; break;          /* COMPUTE_CAPABILITY_MINOR */
    case 102: *v = 1; break;         /* VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED */
    case 132: *v = 1; break;         /* MULTICAST_SUPPORTED */
    default: *v = 0;
  }
  return 0;
}
CUresult cuDeviceTotalMem_v2(size_t* b, CUdevice d) { (void)d; *b = (size_t)180 << 30; return 0; }
CUresult cuDeviceGetPCIBusId(char* s, int len, CUdevice d) { snprintf(s, len, "0000:%02X:00.0", 0x10 + d); return 0; }
CUresult cuDeviceCanAccessPeer(int* can, CUdevice a, CUdevice b) { *can = (a != b) && !flag("FAKE_CUDA_NO_PEER"); return 0; }
CUresult cuDeviceGetP2PAttribute(int* v, int attr, CUdevice a, CUdevice b) { (void)attr; (void)a; (void)b; *v = 1; return 0; }
CUresult cuDevicePrimaryCtxRetain(CUcontext* c, CUdevice d) { *c = (void*)(long)(d + 1); return 0; }
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice d) { (void)d; return 0; }
CUresult cuCtxPushCurrent_v2(CUcontext c) { cur_dev = (int)(long)c - 1; return 0; }
CUresult cuCtxPopCurrent_v2(CUcontext* c) { *c = 0; return 0; }
CUresult cuMemGetInfo_v2(size_t* fr, size_t* tot) { *tot = (size_t)180 << 30; *fr = ((size_t)170 - cur_dev) << 30; return 0; }
CUresult cuMemGetAllocationGranularity(size_t* g, const void* prop, int opt) { (void)prop; (void)opt; *g = 2u << 20; return 0; }
CUresult cuMemAddressReserve(CUdeviceptr* p, size_t size, size_t al, CUdeviceptr addr, unsigned long long fl) {
  (void)al; (void)addr; (void)fl;
  void* m = aligned_alloc(2u << 20, size);
  if (!m) return 2;
  *p = (CUdeviceptr)m;
  return 0;
}
CUresult cuMemAddressFree(CUdeviceptr p, size_t size) { (void)size; free((void*)p); return 0; }
CUresult cuMemCreate(CUmemGenericAllocationHandle* h, size_t size, const void* prop, unsigned long long fl) {
  (void)size; (void)fl;
  if (flag("FAKE_CUDA_FAIL_CREATE")) return 2;
  /* CUmemAllocationProp: type(int) requestedHandleTypes(int) location{type(int) id(int)} ... */
  *h = 1000 + ((const int*)prop)[3];
  return 0;
}
CUresult cuMemRelease(CUmemGenericAllocationHandle h) { (void)h; return 0; }
/* A shareable handle is a memfd that holds the handle's value: it survives SCM_RIGHTS to another process. */
CUresult cuMemExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, int type, unsigned long long fl) {
  (void)fl;
  if (type != 1 || flag("FAKE_CUDA_FAIL_EXPORT")) return 801;
  int fd = memfd_create("fake_cuda_handle", 0);
  if (fd < 0) return 2;
  if (write(fd, &h, sizeof h) != (ssize_t)sizeof h) { close(fd); return 2; }
  *(int*)out = fd;
  return 0;
}
/* Multicast objects: a handle in its own number range; devices added and blocks bound are only counted. */
typedef struct { unsigned numDevices; size_t size; unsigned long long handleTypes, flags; } FakeMcProp;
static int mc_added = 0, mc_bound = 0;
CUresult cuMulticastGetGranularity(size_t* g, const void* prop, int opt) { (void)prop; (void)opt; *g = 4u << 20; return 0; }
CUresult cuMulticastCreate(CUmemGenericAllocationHandle* h, const void* prop) {
  const FakeMcProp* p = (const FakeMcProp*)prop;
  if (flag("FAKE_CUDA_NO_MULTICAST") || p->numDevices < 2 || (p->size % (4u << 20))) return 801;
  *h = 5000 + p->numDevices;
  return 0;
}
CUresult cuMulticastAddDevice(CUmemGenericAllocationHandle h, CUdevice d) { if (h < 5000 || d < 0 || d >= ndev()) return 1; ++mc_added; return 0; }
CUresult cuMulticastBindMem(CUmemGenericAllocationHandle mc, size_t mo, CUmemGenericAllocationHandle mem, size_t o, size_t size, unsigned long long fl) {
  (void)mo; (void)o; (void)fl;
  if (mc < 5000 || mem < 1000 || mem >= 5000 || (size % (4u << 20)) || mc_added < (int)(mc - 5000)) return 1;   /* every device first */
  ++mc_bound;
  return 0;
}
CUresult cuMulticastUnbind(CUmemGenericAllocationHandle mc, CUdevice d, size_t mo, size_t size) { (void)mc; (void)d; (void)mo; (void)size; --mc_bound; return 0; }
CUresult cuMemImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, int type) {
  if (type != 1) return 801;
  int fd = (int)(long)os_handle;
  if (pread(fd, h, sizeof *h, 0) != (ssize_t)sizeof *h) return 1;
  return 0;
}
CUresult cuMemMap(CUdeviceptr p, size_t size, size_t off, CUmemGenericAllocationHandle h, unsigned long long fl) {
  (void)off; (void)fl;
  if (nmaps >= 64) return 2;
  maps[nmaps].va = p; maps[nmaps].size = size; maps[nmaps].device = h >= 5000 ? -2 : (int)(h - 1000); ++nmaps;
  return 0;
}
CUresult cuMemUnmap(CUdeviceptr p, size_t size) {
  (void)size;
  for (int i = 0; i < nmaps; ++i) if (maps[i].va == p) { maps[i] = maps[--nmaps]; break; }
  return 0;
}
CUresult cuMemSetAccess(CUdeviceptr p, size_t size, const void* desc, size_t n) { (void)p; (void)size; (void)desc; (void)n; return 0; }
CUresult cuPointerGetAttribute(void* out, int attr, CUdeviceptr p) {
  (void)attr;
  for (int i = 0; i < nmaps; ++i)
    if (p >= maps[i].va && p < maps[i].va + maps[i].size) { *(int*)out = maps[i].device; return 0; }
  return 1;
}
