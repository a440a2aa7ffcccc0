// Virtual-memory slab: one reserved device address range whose pieces are backed by physical memory only while they are
// mapped. A block of weights keeps its address for the life of the slab, so kernels, tensor views and captured CUDA graphs
// that name the address stay valid while the physical pages behind cold blocks are released and later re-created
// (reserve -> create / map / set-access per block -> unmap / release). The counterpart of the reference's
// serenitymojo/offload/vmm_slab.mojo:44-171. Driver entry points are looked up at run time (no link against libcuda).
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/library.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>

namespace {

template <typename F> F driver_fn(const char* name) {
  void* f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<F>(f);
}

struct Api {
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  bool ok = false;
};

const Api& api() {
  static Api a = [] {
    Api x;
    cudaFree(nullptr);   // a current context for the driver calls
    x.reserve = driver_fn<decltype(x.reserve)>("cuMemAddressReserve");
    x.addr_free = driver_fn<decltype(x.addr_free)>("cuMemAddressFree");
    x.create = driver_fn<decltype(x.create)>("cuMemCreate");
    x.release = driver_fn<decltype(x.release)>("cuMemRelease");
    x.map = driver_fn<decltype(x.map)>("cuMemMap");
    x.unmap = driver_fn<decltype(x.unmap)>("cuMemUnmap");
    x.set_access = driver_fn<decltype(x.set_access)>("cuMemSetAccess");
    x.granularity = driver_fn<decltype(x.granularity)>("cuMemGetAllocationGranularity");
    x.ok = x.reserve && x.addr_free && x.create && x.release && x.map && x.unmap && x.set_access && x.granularity;
    return x;
  }();
  return a;
}

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

struct Region {
  CUmemGenericAllocationHandle handle;
  size_t bytes;
};

struct Slab {
  int device = 0;
  CUdeviceptr base = 0;
  size_t size = 0, gran = 0, mapped = 0;
  std::map<size_t, Region> regions;   // offset -> mapped region
};

std::mutex g_mu;
std::map<int64_t, std::unique_ptr<Slab>> g_slabs;
int64_t g_next = 1;

void check(CUresult r, const char* what) { TORCH_CHECK(r == CUDA_SUCCESS, "vmm_slab: ", what, " failed with CUresult ", (int)r); }

Slab& slab_of(int64_t h) {
  auto it = g_slabs.find(h);
  TORCH_CHECK(it != g_slabs.end(), "vmm_slab: unknown slab handle ", h);
  return *it->second;
}

int64_t vmm_granularity(int64_t device) {
  TORCH_CHECK(api().ok, "vmm_slab: the driver's virtual-memory entry points are not available");
  size_t g = 0;
  CUmemAllocationProp p = prop_for((int)device);
  check(api().granularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "cuMemGetAllocationGranularity");
  return (int64_t)g;
}

// reserves `bytes` (rounded up to the allocation granularity) of device address space; nothing is backed yet
int64_t vmm_slab_create(int64_t bytes, int64_t device) {
  TORCH_CHECK(bytes > 0, "vmm_slab: size must be positive");
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  auto s = std::make_unique<Slab>();
  s->device = (int)device;
  s->gran = (size_t)vmm_granularity(device);
  s->size = ((size_t)bytes + s->gran - 1) / s->gran * s->gran;
  check(api().reserve(&s->base, s->size, s->gran, 0, 0), "cuMemAddressReserve");
  std::lock_guard<std::mutex> lk(g_mu);
  int64_t h = g_next++;
  g_slabs[h] = std::move(s);
  return h;
}

// backs [offset, offset + bytes) with fresh physical memory (offset and bytes multiples of the granularity)
void vmm_slab_map(int64_t h, int64_t offset, int64_t bytes) {
  std::lock_guard<std::mutex> lk(g_mu);
  Slab& s = slab_of(h);
  TORCH_CHECK(offset >= 0 && bytes > 0 && (size_t)offset % s.gran == 0 && (size_t)bytes % s.gran == 0 && (size_t)(offset + bytes) <= s.size,
              "vmm_slab: region must be granularity-aligned and inside the slab");
  for (auto& kv : s.regions)
    TORCH_CHECK((size_t)offset >= kv.first + kv.second.bytes || (size_t)(offset + bytes) <= kv.first, "vmm_slab: region overlaps a mapped one");
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)s.device);
  CUmemAllocationProp p = prop_for(s.device);
  Region r{0, (size_t)bytes};
  check(api().create(&r.handle, r.bytes, &p, 0), "cuMemCreate");
  CUresult e = api().map(s.base + offset, r.bytes, 0, r.handle, 0);
  if (e != CUDA_SUCCESS) { api().release(r.handle); check(e, "cuMemMap"); }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = s.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  e = api().set_access(s.base + offset, r.bytes, &acc, 1);
  if (e != CUDA_SUCCESS) { api().unmap(s.base + offset, r.bytes); api().release(r.handle); check(e, "cuMemSetAccess"); }
  s.regions[(size_t)offset] = r;
  s.mapped += r.bytes;
}

// releases the physical memory behind the region mapped at `offset`; the caller has made sure no work still uses it
void vmm_slab_unmap(int64_t h, int64_t offset) {
  std::lock_guard<std::mutex> lk(g_mu);
  Slab& s = slab_of(h);
  auto it = s.regions.find((size_t)offset);
  TORCH_CHECK(it != s.regions.end(), "vmm_slab: nothing is mapped at offset ", offset);
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)s.device);
  check(api().unmap(s.base + offset, it->second.bytes), "cuMemUnmap");
  check(api().release(it->second.handle), "cuMemRelease");
  s.mapped -= it->second.bytes;
  s.regions.erase(it);
}

// a uint8 view of a mapped range (the tensor does not own the memory)
at::Tensor vmm_slab_tensor(int64_t h, int64_t offset, int64_t bytes) {
  std::lock_guard<std::mutex> lk(g_mu);
  Slab& s = slab_of(h);
  bool inside = false;
  for (auto& kv : s.regions)
    if ((size_t)offset >= kv.first && (size_t)(offset + bytes) <= kv.first + kv.second.bytes) inside = true;
  TORCH_CHECK(inside && bytes > 0, "vmm_slab: the requested view is not inside one mapped region");
  return at::from_blob(reinterpret_cast<void*>(s.base + offset), {bytes},
                       at::TensorOptions().dtype(at::kByte).device(at::kCUDA, (c10::DeviceIndex)s.device));
}

std::vector<int64_t> vmm_slab_info(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  Slab& s = slab_of(h);
  return {(int64_t)s.base, (int64_t)s.size, (int64_t)s.gran, (int64_t)s.mapped, (int64_t)s.regions.size()};
}

void vmm_slab_destroy(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  Slab& s = slab_of(h);
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)s.device);
  for (auto& kv : s.regions) {
    api().unmap(s.base + kv.first, kv.second.bytes);
    api().release(kv.second.handle);
  }
  api().addr_free(s.base, s.size);
  g_slabs.erase(h);
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(mdb200, m) {
  m.def("vmm_granularity", &vmm_granularity);
  m.def("vmm_slab_create", &vmm_slab_create);
  m.def("vmm_slab_map", &vmm_slab_map);
  m.def("vmm_slab_unmap", &vmm_slab_unmap);
  m.def("vmm_slab_tensor", &vmm_slab_tensor);
  m.def("vmm_slab_info", &vmm_slab_info);
  m.def("vmm_slab_destroy", &vmm_slab_destroy);
}
