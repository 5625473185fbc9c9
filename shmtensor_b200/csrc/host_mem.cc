// Host memory substrate: POSIX shared memory, mmap'ed .npy files and host
// registration.  Host-only code; the kernels read these buffers through UVA.
// Behaviour follows the reference's include/shm_memory.h:6-49, include/utils.h:5-13,
// src/mmap_tensor.cc:10-55, src/cnpy.cc:18-86 and src/cache_feature_fetch.cu:6-13,
// except that failures come back as status codes instead of aborting.
#include <cuda_runtime.h>
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sched.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <string>
#include <thread>
#include <vector>

#include "shmt.h"

namespace shmt {
void set_error(const char* fmt, ...);
}
using shmt::set_error;

namespace {

int register_host(void* ptr, size_t size, unsigned flags, const char* who) {
  cudaError_t e = cudaHostRegister(ptr, size, flags);
  if (e != cudaSuccess) {
    set_error("%s: cudaHostRegister(%zu bytes) failed: %s", who, size, cudaGetErrorString(e));
    return SHMT_ERR_CUDA;
  }
  return SHMT_OK;
}

int map_shared(const char* who, const char* name, int64_t size, int pin_memory, bool create,
               int64_t* out_ptr, int64_t* out_fd, bool exclusive = false) {
  if (!name || !out_ptr || !out_fd || size <= 0) {
    set_error("%s: bad argument (name/size/out)", who);
    return SHMT_ERR_INVALID;
  }
  const int flag = create ? (O_RDWR | O_CREAT | (exclusive ? O_EXCL : 0)) : O_RDWR;
  const int fd = shm_open(name, flag, S_IRUSR | S_IWUSR);
  if (fd == -1) {
    if (exclusive && errno == EEXIST)
      set_error("%s: a segment named %s already exists", who, name);
    else
      set_error("%s: fail to open %s: %s", who, name, strerror(errno));
    return SHMT_ERR_OS;
  }
  if (create && ftruncate(fd, (off_t)size) == -1) {
    set_error("%s: failed to truncate %s to %lld bytes: %s", who, name, (long long)size,
              strerror(errno));
    close(fd);
    shm_unlink(name);
    return SHMT_ERR_OS;
  }
  void* ptr = mmap(nullptr, (size_t)size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (ptr == MAP_FAILED) {
    set_error("%s: failed to map shared memory %s: %s", who, name, strerror(errno));
    close(fd);
    if (create) shm_unlink(name);
    return SHMT_ERR_OS;
  }
  if (pin_memory) {
    // Portable: usable from every GPU of the process, not only the one current now (the
    // reference registers with the default flag, which binds to the current context)
    if (int rc = register_host(ptr, (size_t)size, cudaHostRegisterPortable, who)) {
      munmap(ptr, (size_t)size);
      close(fd);
      if (create) shm_unlink(name);
      return rc;
    }
  }
  *out_ptr = (int64_t)(intptr_t)ptr;
  *out_fd = fd;
  return SHMT_OK;
}

// Value of a key in the Python-dict text of an .npy header, e.g. 'descr': '<f4'.
bool find_after(const std::string& h, const char* key, size_t* pos) {
  const size_t k = h.find(key);
  if (k == std::string::npos) return false;
  const size_t c = h.find(':', k);
  if (c == std::string::npos) return false;
  size_t p = c + 1;
  while (p < h.size() && h[p] == ' ') ++p;
  *pos = p;
  return true;
}


// ---- NUMA placement of host tables -------------------------------------------------------
// GPUs read a host table over their own PCIe links, but all those reads end at the memory
// controllers of whichever node holds the pages; a table first-touched by one process sits on
// one node, and the GPUs of the other socket then share the inter-socket link.

// Parses a kernel list such as "0-3,8,10-11" into ids.
std::vector<int> parse_id_list(const char* path) {
  std::vector<int> out;
  FILE* f = fopen(path, "r");
  if (!f) return out;
  char buf[4096];
  if (fgets(buf, sizeof(buf), f)) {
    const char* p = buf;
    while (*p) {
      while (*p && (*p < '0' || *p > '9')) ++p;
      if (!*p) break;
      int a = 0;
      while (*p >= '0' && *p <= '9') a = a * 10 + (*p++ - '0');
      int b = a;
      if (*p == '-') {
        ++p;
        b = 0;
        while (*p >= '0' && *p <= '9') b = b * 10 + (*p++ - '0');
      }
      for (int v = a; v <= b && out.size() < 4096; ++v) out.push_back(v);
    }
  }
  fclose(f);
  return out;
}

std::vector<int> memory_nodes() {
  std::vector<int> nodes = parse_id_list("/sys/devices/system/node/has_memory");
  if (nodes.empty()) nodes = parse_id_list("/sys/devices/system/node/online");
  if (nodes.empty()) nodes.push_back(0);
  return nodes;
}

// Touch (write one zero byte per 4 KB of) the pieces of [base, base+bytes) that `node` should
// hold, from a thread restricted to that node's CPUs, so that first-touch allocation puts
// them there.  `every` > 1: node takes chunk c when c % every == which (coarse interleave).
bool first_touch_on_node(char* base, size_t bytes, int node, size_t chunk, int every, int which) {
  char path[128];
  snprintf(path, sizeof(path), "/sys/devices/system/node/node%d/cpulist", node);
  const std::vector<int> cpus = parse_id_list(path);
  cpu_set_t allowed, want;
  CPU_ZERO(&want);
  if (sched_getaffinity(0, sizeof(allowed), &allowed) != 0) return false;
  int usable = 0;
  for (int c : cpus)
    if (c < CPU_SETSIZE && CPU_ISSET(c, &allowed)) {
      CPU_SET(c, &want);
      ++usable;
    }
  if (usable == 0) return false;  // this process may not run on that node's cores
  bool ok = true;
  std::thread worker([&] {
    if (sched_setaffinity(0, sizeof(want), &want) != 0) {
      ok = false;
      return;
    }
    for (size_t off = 0, c = 0; off < bytes; off += chunk, ++c) {
      if ((int)(c % (size_t)every) != which) continue;
      const size_t end = off + chunk < bytes ? off + chunk : bytes;
      for (size_t q = off; q < end; q += 4096) *reinterpret_cast<volatile char*>(base + q) = 0;
    }
  });
  worker.join();
  return ok;
}

}  // namespace

extern "C" {

int shmt_shm_create(const char* name, int64_t size, int pin_memory, int64_t* out_ptr,
                    int64_t* out_fd) {
  return map_shared("shmt_shm_create", name, size, pin_memory, true, out_ptr, out_fd);
}

int shmt_shm_create_excl(const char* name, int64_t size, int pin_memory, int64_t* out_ptr,
                         int64_t* out_fd) {
  return map_shared("shmt_shm_create_excl", name, size, pin_memory, true, out_ptr, out_fd,
                    /*exclusive=*/true);
}

int shmt_shm_unlink(const char* name) {
  if (!name) {
    set_error("shmt_shm_unlink: name is null");
    return SHMT_ERR_INVALID;
  }
  if (shm_unlink(name) == -1 && errno != ENOENT) {
    set_error("shmt_shm_unlink: %s: %s", name, strerror(errno));
    return SHMT_ERR_OS;
  }
  return SHMT_OK;
}

int shmt_shm_open(const char* name, int64_t size, int pin_memory, int64_t* out_ptr,
                  int64_t* out_fd) {
  return map_shared("shmt_shm_open", name, size, pin_memory, false, out_ptr, out_fd);
}

int shmt_shm_release(const char* name, int64_t size, int64_t ptr, int64_t fd, int pin_memory) {
  if (!name || !ptr) {
    set_error("shmt_shm_release: bad argument");
    return SHMT_ERR_INVALID;
  }
  int rc = SHMT_OK;
  if (pin_memory) {
    cudaError_t e = cudaHostUnregister((void*)(intptr_t)ptr);
    if (e != cudaSuccess) {
      set_error("shmt_shm_release: cudaHostUnregister failed: %s", cudaGetErrorString(e));
      rc = SHMT_ERR_CUDA;
    }
  }
  if (munmap((void*)(intptr_t)ptr, (size_t)size) == -1) {
    set_error("shmt_shm_release: munmap failed: %s", strerror(errno));
    rc = SHMT_ERR_OS;
  }
  close((int)fd);
  shm_unlink(name);
  return rc;
}

int shmt_shm_exists(const char* name) {
  if (!name) return 0;
  const int fd = shm_open(name, O_RDONLY, S_IRUSR | S_IWUSR);
  if (fd >= 0) {
    close(fd);
    return 1;
  }
  return 0;
}

int shmt_npy_open(const char* path, int flags, shmt_npy_info* out) {
  if (!path || !out) {
    set_error("shmt_npy_open: bad argument");
    return SHMT_ERR_INVALID;
  }
  const int pin_memory = flags & SHMT_NPY_PIN;
  const bool read_only = (flags & SHMT_NPY_READONLY) != 0;
  memset(out, 0, sizeof(*out));
  const int fd = open(path, read_only ? O_RDONLY : O_RDWR, S_IRUSR | S_IWUSR);
  if (fd == -1) {
    set_error("npy_load: Unable to open file %s: %s", path, strerror(errno));
    return SHMT_ERR_OS;
  }
  struct stat sb;
  if (fstat(fd, &sb) == -1 || sb.st_size < 10) {
    set_error("shmt_npy_open: %s is not an .npy file", path);
    close(fd);
    return SHMT_ERR_OS;
  }
  const size_t file_size = (size_t)sb.st_size;
  void* base = mmap(nullptr, file_size, read_only ? PROT_READ : (PROT_READ | PROT_WRITE), MAP_SHARED,
                    fd, 0);
  if (base == MAP_FAILED) {
    set_error("shmt_npy_open: mmap of %s failed: %s", path, strerror(errno));
    close(fd);
    return SHMT_ERR_OS;
  }
  const unsigned char* b = static_cast<const unsigned char*>(base);
  auto fail = [&](const char* why) {
    set_error("parse_npy_header: %s (%s)", why, path);
    munmap(base, file_size);
    close(fd);
    return SHMT_ERR_INVALID;
  };
  if (memcmp(b, "\x93NUMPY", 6) != 0) return fail("bad magic");
  const int major = b[6];
  size_t hlen = 0, hstart = 0;
  if (major == 1) {
    hlen = b[8] | (b[9] << 8);
    hstart = 10;
  } else if (major == 2 || major == 3) {
    if (file_size < 12) return fail("truncated header");
    hlen = (size_t)b[8] | ((size_t)b[9] << 8) | ((size_t)b[10] << 16) | ((size_t)b[11] << 24);
    hstart = 12;
  } else {
    return fail("unsupported .npy version");
  }
  if (hstart + hlen > file_size) return fail("truncated header");
  const std::string h(reinterpret_cast<const char*>(b + hstart), hlen);

  size_t p = 0;
  if (!find_after(h, "fortran_order", &p))
    return fail("failed to find header keyword: 'fortran_order'");
  out->fortran_order = h.compare(p, 4, "True") == 0;
  if (!find_after(h, "descr", &p)) return fail("failed to find header keyword: 'descr'");
  if (p >= h.size() || (h[p] != '\'' && h[p] != '"')) return fail("structured dtypes are not supported");
  const size_t q = h.find(h[p], p + 1);
  if (q == std::string::npos || q - p - 1 >= sizeof(out->descr)) return fail("bad descr");
  memcpy(out->descr, h.data() + p + 1, q - p - 1);
  if (!find_after(h, "shape", &p)) return fail("failed to find header keyword: 'shape'");
  const size_t lp = h.find('(', p), rp = h.find(')', p);
  if (lp == std::string::npos || rp == std::string::npos || rp < lp)
    return fail("failed to find header keyword: '(' or ')'");
  int ndim = 0;
  size_t i = lp + 1;
  while (i < rp) {
    while (i < rp && (h[i] < '0' || h[i] > '9')) ++i;
    if (i >= rp) break;
    int64_t v = 0;
    while (i < rp && h[i] >= '0' && h[i] <= '9') v = v * 10 + (h[i++] - '0');
    if (ndim >= 8) return fail("more than 8 dimensions");
    out->shape[ndim++] = v;
  }
  out->ndim = ndim;
  out->data_offset = (int64_t)(hstart + hlen);
  out->file_size = (int64_t)file_size;
  out->ptr = (int64_t)(intptr_t)base;
  out->fd = fd;
  if (pin_memory) {
    // like the reference, register the whole mapping (header included)
    // a mapping without write permission can only be registered as read-only for the device too
    const unsigned reg = cudaHostRegisterPortable | (read_only ? cudaHostRegisterReadOnly : 0u);
    if (int rc = register_host(base, file_size, reg, "shmt_npy_open")) {
      munmap(base, file_size);
      close(fd);
      return rc;
    }
  }
  return SHMT_OK;
}

int shmt_npy_close(int64_t size, int64_t ptr, int64_t fd, int pin_memory) {
  int rc = SHMT_OK;
  if (pin_memory) {
    cudaError_t e = cudaHostUnregister((void*)(intptr_t)ptr);
    if (e != cudaSuccess) {
      set_error("shmt_npy_close: cudaHostUnregister failed: %s", cudaGetErrorString(e));
      rc = SHMT_ERR_CUDA;
    }
  }
  if (munmap((void*)(intptr_t)ptr, (size_t)size) == -1) {
    set_error("shmt_npy_close: munmap failed: %s", strerror(errno));
    rc = SHMT_ERR_OS;
  }
  close((int)fd);
  return rc;
}

int shmt_host_register(void* ptr, int64_t nbytes) {
  if (!ptr || nbytes <= 0) {
    set_error("shmt_host_register: bad argument");
    return SHMT_ERR_INVALID;
  }
  return register_host(ptr, (size_t)nbytes, cudaHostRegisterPortable, "shmt_host_register");
}

int shmt_host_prefault(void* ptr, int64_t nbytes, int n_threads) {
  if (!ptr || nbytes <= 0) {
    set_error("shmt_host_prefault: bad argument");
    return SHMT_ERR_INVALID;
  }
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 64) n_threads = 64;
  char* base = static_cast<char*>(ptr);
  const size_t total = (size_t)nbytes;
  // slices of whole 2 MB pieces, one thread each: a fresh shared mapping has no pages yet, and
  // one thread asking the kernel for them page by page manages only a few GB/s
  const size_t piece = (size_t)2 << 20;
  const size_t n_pieces = (total + piece - 1) / piece;
  std::vector<std::thread> workers;
  for (int t = 0; t < n_threads; ++t) {
    workers.emplace_back([=] {
      for (size_t p = (size_t)t; p < n_pieces; p += (size_t)n_threads) {
        const size_t lo = p * piece, hi = lo + piece < total ? lo + piece : total;
        for (size_t q = lo; q < hi; q += 4096) *reinterpret_cast<volatile char*>(base + q) = 0;
      }
    });
  }
  for (auto& w : workers) w.join();
  return SHMT_OK;
}

int shmt_host_numa_nodes(void) { return (int)memory_nodes().size(); }

int shmt_host_numa_place(void* ptr, int64_t nbytes, int policy, int node) {
  if (!ptr || nbytes <= 0 || ((uintptr_t)ptr & 4095) != 0) {
    set_error("shmt_host_numa_place: needs a page-aligned range");
    return SHMT_ERR_INVALID;
  }
  const std::vector<int> nodes = memory_nodes();
  if (policy != SHMT_NUMA_INTERLEAVE && policy != SHMT_NUMA_BIND) {
    set_error("shmt_host_numa_place: policy %d is neither SHMT_NUMA_INTERLEAVE nor SHMT_NUMA_BIND", policy);
    return SHMT_ERR_INVALID;
  }
  if (policy == SHMT_NUMA_BIND) {
    bool known = false;
    for (int n : nodes) known = known || n == node;
    if (!known) {
      set_error("shmt_host_numa_place: node %d holds no memory on this machine", node);
      return SHMT_ERR_INVALID;
    }
  }
  if (nodes.size() <= 1) return SHMT_OK;  // one node: every placement is the same
  // 1. ask the kernel: a policy on the range (for a shared mapping it belongs to the segment, so
  //    every process that maps it allocates the same way); pages already present are moved
  unsigned long mask[16] = {0};
  for (int n : nodes)
    if (n < 1024 && (policy == SHMT_NUMA_INTERLEAVE || n == node)) mask[n / 64] |= 1UL << (n % 64);
  const int kMpolBind = 2, kMpolInterleave = 3, kMfMove = 2;
  const long rc = syscall(SYS_mbind, ptr, (unsigned long)nbytes,
                          policy == SHMT_NUMA_BIND ? kMpolBind : kMpolInterleave, mask, 1025UL,
                          kMfMove);
  if (rc == 0) return SHMT_OK;
  // 2. containers often forbid mbind: fall back to first touch from threads that run on the
  //    wanted node (only pages not touched yet end up there)
  const int err = errno;
  char* base = static_cast<char*>(ptr);
  bool ok = true;
  if (policy == SHMT_NUMA_BIND) {
    ok = first_touch_on_node(base, (size_t)nbytes, node, (size_t)nbytes, 1, 0);
  } else {
    for (size_t i = 0; i < nodes.size() && ok; ++i)
      ok = first_touch_on_node(base, (size_t)nbytes, nodes[i], (size_t)2 << 20, (int)nodes.size(), (int)i);
  }
  if (!ok) {
    set_error("shmt_host_numa_place: mbind failed (%s) and this process cannot run on the wanted node's cores",
              strerror(err));
    return SHMT_ERR_OS;
  }
  return SHMT_OK;
}

int shmt_host_unregister(void* ptr) {
  cudaError_t e = cudaHostUnregister(ptr);
  if (e != cudaSuccess) {
    set_error("shmt_host_unregister: %s", cudaGetErrorString(e));
    return SHMT_ERR_CUDA;
  }
  return SHMT_OK;
}

}  // extern "C"
