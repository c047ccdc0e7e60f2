// shm.cc -- see shm.h.
#include "shm.h"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>

#include "base.h"

namespace fcx {

namespace {
constexpr uint64_t kRingMagic = 0x464358524e4731ull; // "FCXRNG1"
}

flagcxResult_t ShmRing::create(const std::string &name, size_t capacity) {
  close();
  if (capacity < 4096 || (capacity & (capacity - 1))) return flagcxInvalidArgument;
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) {
    FCX_INFO(SUB_SHM, "shm_open(%s) failed: %s", name.c_str(), strerror(errno));
    return flagcxSystemError;
  }
  const size_t bytes = sizeof(Header) + capacity;
  // posix_fallocate reserves the pages now: a full /dev/shm is an error here, not a SIGBUS later
  int rc = posix_fallocate(fd, 0, (off_t)bytes);
  if (rc != 0) {
    FCX_INFO(SUB_SHM, "no room for %zu bytes of shared memory (%s): %s", bytes, name.c_str(), strerror(rc));
    ::close(fd);
    shm_unlink(name.c_str());
    return flagcxSystemError;
  }
  void *p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) {
    shm_unlink(name.c_str());
    return flagcxSystemError;
  }
  hdr_ = new (p) Header();
  hdr_->head.store(0, std::memory_order_relaxed);
  hdr_->tail.store(0, std::memory_order_relaxed);
  hdr_->capacity = capacity;
  data_ = (char *)p + sizeof(Header);
  mapBytes_ = bytes;
  name_ = name;
  std::atomic_thread_fence(std::memory_order_release);
  hdr_->magic = kRingMagic;
  return flagcxSuccess;
}

flagcxResult_t ShmRing::open(const std::string &name) {
  close();
  int fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) return flagcxSystemError;
  struct stat st;
  if (fstat(fd, &st) != 0 || (size_t)st.st_size < sizeof(Header) + 4096) {
    ::close(fd);
    return flagcxSystemError;
  }
  void *p = mmap(nullptr, (size_t)st.st_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) return flagcxSystemError;
  Header *h = (Header *)p;
  if (h->magic != kRingMagic || sizeof(Header) + h->capacity != (size_t)st.st_size) {
    munmap(p, (size_t)st.st_size);
    return flagcxInternalError;
  }
  hdr_ = h;
  data_ = (char *)p + sizeof(Header);
  mapBytes_ = (size_t)st.st_size;
  shm_unlink(name.c_str()); // both sides are attached: the name has done its job
  return flagcxSuccess;
}

void ShmRing::close() {
  if (hdr_) munmap((void *)hdr_, mapBytes_);
  hdr_ = nullptr;
  data_ = nullptr;
  mapBytes_ = 0;
  if (!name_.empty()) shm_unlink(name_.c_str()); // harmless if the receiver removed it already
  name_.clear();
}

size_t ShmRing::write(const void *src, size_t n) {
  const uint64_t cap = hdr_->capacity;
  const uint64_t head = hdr_->head.load(std::memory_order_relaxed);
  const uint64_t tail = hdr_->tail.load(std::memory_order_acquire);
  const size_t room = (size_t)(cap - (head - tail));
  n = std::min(n, room);
  if (n == 0) return 0;
  const size_t at = (size_t)(head & (cap - 1));
  const size_t first = std::min(n, (size_t)cap - at);
  memcpy(data_ + at, src, first);
  if (n > first) memcpy(data_, (const char *)src + first, n - first);
  hdr_->head.store(head + n, std::memory_order_release);
  return n;
}

size_t ShmRing::read(void *dst, size_t n) {
  const uint64_t cap = hdr_->capacity;
  const uint64_t tail = hdr_->tail.load(std::memory_order_relaxed);
  const uint64_t head = hdr_->head.load(std::memory_order_acquire);
  n = std::min(n, (size_t)(head - tail));
  if (n == 0) return 0;
  const size_t at = (size_t)(tail & (cap - 1));
  const size_t first = std::min(n, (size_t)cap - at);
  memcpy(dst, data_ + at, first);
  if (n > first) memcpy((char *)dst + first, data_, n - first);
  hdr_->tail.store(tail + n, std::memory_order_release);
  return n;
}

bool processIsDead(int pid) {
  char path[64];
  snprintf(path, sizeof path, "/proc/%d/stat", pid);
  FILE *f = fopen(path, "r");
  if (!f) return errno == ENOENT;
  char buf[512];
  size_t got = fread(buf, 1, sizeof buf - 1, f);
  fclose(f);
  buf[got] = 0;
  // "pid (comm) S ...": the state letter follows the LAST ')' (comm may contain any character)
  const char *rp = strrchr(buf, ')');
  if (!rp || !rp[1] || !rp[2]) return false;
  const char state = rp[2];
  return state == 'Z' || state == 'X' || state == 'x';
}

} // namespace fcx
