// Virtual-memory-mapped tensors over a shared pool of physical pages.
//
// A model's weights and KV cache live in virtual address ranges ("XTensor") that are reserved once
// at their maximum size; physical pages of a fixed size are taken from a pool shared by every model
// on the device and mapped in on demand.  Putting a model to sleep unmaps its ranges and gives the
// pages back; another model can wake up on the same pages; the virtual addresses (and so every
// tensor and captured CUDA graph that points into them) stay valid across the cycle.
//
// Parity: xllm/core/framework/xtensor/{phy_page_pool,page_allocator,xtensor_allocator}.cpp and
// xllm/core/platform/vmm_api.cpp (cuMemCreate / cuMemAddressReserve / cuMemMap / cuMemSetAccess).
//
// The CUDA driver is reached through a function table resolved with dlopen at run time, so the
// module loads on machines without a driver; `fake_driver()` implements the same table on host
// memory (memfd pages mapped with MAP_FIXED into a PROT_NONE reservation), which keeps the
// semantics the pool relies on: a page keeps its contents while it is unmapped, and touching an
// unmapped part of a range faults.
#pragma once
#include <dlfcn.h>
#include <sys/mman.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#if __has_include(<cuda.h>)
#include <cuda.h>
#define XLLM_HAVE_CUDA_H 1
#endif

namespace xllm {

struct VmmDriver {
  const char* name;
  int (*granularity)(size_t* out, int device);
  int (*create)(uint64_t* handle, size_t size, int device);
  int (*release)(uint64_t handle);
  int (*reserve)(uint64_t* ptr, size_t size, size_t align);
  int (*free_range)(uint64_t ptr, size_t size);
  int (*map)(uint64_t ptr, size_t size, uint64_t handle);
  int (*unmap)(uint64_t ptr, size_t size);
  int (*set_access)(uint64_t ptr, size_t size, int device);
};

// ------------------------------------------------------------------------------------ host fake
namespace vmm_fake {
inline int granularity(size_t* out, int) { *out = 64 * 1024; return 0; }
inline int create(uint64_t* handle, size_t size, int) {
  int fd = memfd_create("xllm_vmm_page", 0);
  if (fd < 0) return 1;
  if (ftruncate(fd, (off_t)size) != 0) { close(fd); return 2; }
  *handle = (uint64_t)fd + 1;      // 0 stays "no handle"
  return 0;
}
inline int release(uint64_t handle) { return close((int)(handle - 1)) == 0 ? 0 : 1; }
inline int reserve(uint64_t* ptr, size_t size, size_t) {
  void* p = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return 1;
  *ptr = (uint64_t)p;
  return 0;
}
inline int free_range(uint64_t ptr, size_t size) { return munmap((void*)ptr, size) == 0 ? 0 : 1; }
inline int map(uint64_t ptr, size_t size, uint64_t handle) {
  void* p = mmap((void*)ptr, size, PROT_NONE, MAP_SHARED | MAP_FIXED, (int)(handle - 1), 0);
  return p == MAP_FAILED ? 1 : 0;
}
inline int unmap(uint64_t ptr, size_t size) {
  void* p = mmap((void*)ptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
  return p == MAP_FAILED ? 1 : 0;
}
inline int set_access(uint64_t ptr, size_t size, int) {
  return mprotect((void*)ptr, size, PROT_READ | PROT_WRITE) == 0 ? 0 : 1;
}
}  // namespace vmm_fake

inline const VmmDriver* fake_driver() {
  static const VmmDriver d{"host-fake",        vmm_fake::granularity, vmm_fake::create,
                           vmm_fake::release,  vmm_fake::reserve,     vmm_fake::free_range,
                           vmm_fake::map,      vmm_fake::unmap,       vmm_fake::set_access};
  return &d;
}

// ------------------------------------------------------------------------------------ CUDA driver
#ifdef XLLM_HAVE_CUDA_H
namespace vmm_cuda {
struct Api {
  CUresult (*cuInit)(unsigned);
  CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
  CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
  CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
  CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  bool ok = false;
};
inline Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    auto sym = [&](const char* n) { return dlsym(h, n); };
#define XLLM_SYM(field, name) a.field = reinterpret_cast<decltype(a.field)>(sym(name))
    XLLM_SYM(cuInit, "cuInit");
    XLLM_SYM(cuMemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    XLLM_SYM(cuMemCreate, "cuMemCreate");
    XLLM_SYM(cuMemRelease, "cuMemRelease");
    XLLM_SYM(cuMemAddressReserve, "cuMemAddressReserve");
    XLLM_SYM(cuMemAddressFree, "cuMemAddressFree");
    XLLM_SYM(cuMemMap, "cuMemMap");
    XLLM_SYM(cuMemUnmap, "cuMemUnmap");
    XLLM_SYM(cuMemSetAccess, "cuMemSetAccess");
#undef XLLM_SYM
    a.ok = a.cuInit && a.cuMemGetAllocationGranularity && a.cuMemCreate && a.cuMemRelease && a.cuMemAddressReserve &&
           a.cuMemAddressFree && a.cuMemMap && a.cuMemUnmap && a.cuMemSetAccess && a.cuInit(0) == CUDA_SUCCESS;
  });
  return a;
}
inline CUmemAllocationProp prop(int device) {
  CUmemAllocationProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}
inline int granularity(size_t* out, int device) {
  auto p = prop(device);
  return (int)api().cuMemGetAllocationGranularity(out, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
}
inline int create(uint64_t* handle, size_t size, int device) {
  auto p = prop(device);
  CUmemGenericAllocationHandle h = 0;
  int rc = (int)api().cuMemCreate(&h, size, &p, 0);
  *handle = (uint64_t)h;
  return rc;
}
inline int release(uint64_t handle) { return (int)api().cuMemRelease((CUmemGenericAllocationHandle)handle); }
inline int reserve(uint64_t* ptr, size_t size, size_t align) {
  CUdeviceptr p = 0;
  int rc = (int)api().cuMemAddressReserve(&p, size, align, 0, 0);
  *ptr = (uint64_t)p;
  return rc;
}
inline int free_range(uint64_t ptr, size_t size) { return (int)api().cuMemAddressFree((CUdeviceptr)ptr, size); }
inline int map(uint64_t ptr, size_t size, uint64_t handle) {
  return (int)api().cuMemMap((CUdeviceptr)ptr, size, 0, (CUmemGenericAllocationHandle)handle, 0);
}
inline int unmap(uint64_t ptr, size_t size) { return (int)api().cuMemUnmap((CUdeviceptr)ptr, size); }
inline int set_access(uint64_t ptr, size_t size, int device) {
  CUmemAccessDesc d;
  std::memset(&d, 0, sizeof(d));
  d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  d.location.id = device;
  d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return (int)api().cuMemSetAccess((CUdeviceptr)ptr, size, &d, 1);
}
}  // namespace vmm_cuda
#endif

/// nullptr when no CUDA driver can be loaded on this machine.
inline const VmmDriver* cuda_driver() {
#ifdef XLLM_HAVE_CUDA_H
  if (!vmm_cuda::api().ok) return nullptr;
  static const VmmDriver d{"cuda",             vmm_cuda::granularity, vmm_cuda::create,
                           vmm_cuda::release,  vmm_cuda::reserve,     vmm_cuda::free_range,
                           vmm_cuda::map,      vmm_cuda::unmap,       vmm_cuda::set_access};
  return &d;
#else
  return nullptr;
#endif
}

// ------------------------------------------------------------------------------------ page pool
class PhyPagePool {
 public:
  PhyPagePool(const VmmDriver* drv, int device, size_t page_bytes, size_t max_pages)
      : drv_(drv), device_(device), max_pages_(max_pages) {
    if (!drv_) throw std::runtime_error("no VMM driver available");
    size_t g = 0;
    check(drv_->granularity(&g, device_), "granularity");
    granularity_ = g ? g : 1;
    page_bytes_ = (page_bytes + granularity_ - 1) / granularity_ * granularity_;
  }
  ~PhyPagePool() {
    for (uint64_t h : free_) drv_->release(h);
  }
  PhyPagePool(const PhyPagePool&) = delete;

  /// A physical page: a recycled one if any is free, else a new allocation up to `max_pages`.
  uint64_t acquire() {
    std::lock_guard<std::mutex> g(mu_);
    if (!free_.empty()) {
      uint64_t h = free_.back();
      free_.pop_back();
      ++in_use_;
      return h;
    }
    if (created_ >= max_pages_) throw std::runtime_error("physical page pool exhausted");
    uint64_t h = 0;
    check(drv_->create(&h, page_bytes_, device_), "create");
    ++created_;
    ++in_use_;
    return h;
  }
  void give_back(uint64_t h) {
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back(h);
    --in_use_;
  }
  /// Returns free pages to the device (e.g. before another process needs the memory).
  size_t trim() {
    std::lock_guard<std::mutex> g(mu_);
    size_t n = free_.size();
    for (uint64_t h : free_) drv_->release(h);
    created_ -= n;
    free_.clear();
    return n;
  }
  size_t page_bytes() const { return page_bytes_; }
  size_t max_pages() const { return max_pages_; }
  size_t pages_created() const { return created_; }
  size_t pages_in_use() const { return in_use_; }
  size_t pages_free() const { return free_.size(); }
  int device() const { return device_; }
  const VmmDriver* driver() const { return drv_; }
  static void check(int rc, const char* what) {
    if (rc != 0) throw std::runtime_error(std::string("vmm ") + what + " failed with code " + std::to_string(rc));
  }

 private:
  const VmmDriver* drv_;
  int device_;
  size_t page_bytes_ = 0, granularity_ = 1, max_pages_;
  size_t created_ = 0, in_use_ = 0;
  std::vector<uint64_t> free_;
  std::mutex mu_;
};

// ------------------------------------------------------------------------------------ mapped range
class XTensor {
 public:
  XTensor(PhyPagePool* pool, size_t virt_bytes) : pool_(pool) {
    const size_t pb = pool_->page_bytes();
    n_slots_ = (virt_bytes + pb - 1) / pb;
    PhyPagePool::check(pool_->driver()->reserve(&base_, n_slots_ * pb, pb), "reserve");
    pages_.assign(n_slots_, 0);
  }
  ~XTensor() {
    release_all();
    pool_->driver()->free_range(base_, n_slots_ * pool_->page_bytes());
  }
  XTensor(const XTensor&) = delete;

  uint64_t ptr() const { return base_; }
  size_t virt_bytes() const { return n_slots_ * pool_->page_bytes(); }
  size_t mapped_bytes() const { return n_mapped_ * pool_->page_bytes(); }
  bool is_mapped(size_t offset) const { return pages_[offset / pool_->page_bytes()] != 0; }

  /// Maps every page that intersects [offset, offset + bytes); already mapped pages are kept.
  void map_range(size_t offset, size_t bytes) {
    if (bytes == 0) return;
    const size_t pb = pool_->page_bytes();
    const size_t a = offset / pb, b = (offset + bytes + pb - 1) / pb;
    if (b > n_slots_) throw std::out_of_range("map_range beyond the reserved range");
    const VmmDriver* d = pool_->driver();
    for (size_t i = a; i < b; ++i) {
      if (pages_[i]) continue;
      uint64_t h = pool_->acquire();
      int rc = d->map(base_ + i * pb, pb, h);
      if (rc == 0) rc = d->set_access(base_ + i * pb, pb, pool_->device());
      if (rc != 0) {
        pool_->give_back(h);
        PhyPagePool::check(rc, "map");
      }
      pages_[i] = h;
      ++n_mapped_;
    }
  }
  /// Unmaps the pages that lie entirely inside [offset, offset + bytes) and returns them to the pool.
  void unmap_range(size_t offset, size_t bytes) {
    const size_t pb = pool_->page_bytes();
    const size_t a = (offset + pb - 1) / pb, b = std::min(n_slots_, (offset + bytes) / pb);
    const VmmDriver* d = pool_->driver();
    for (size_t i = a; i < b; ++i) {
      if (!pages_[i]) continue;
      d->unmap(base_ + i * pb, pb);
      pool_->give_back(pages_[i]);
      pages_[i] = 0;
      --n_mapped_;
    }
  }
  void ensure(size_t bytes) { map_range(0, bytes); }
  void release_all() { unmap_range(0, n_slots_ * pool_->page_bytes()); }

 private:
  PhyPagePool* pool_;
  uint64_t base_ = 0;
  size_t n_slots_ = 0, n_mapped_ = 0;
  std::vector<uint64_t> pages_;
};

}  // namespace xllm
