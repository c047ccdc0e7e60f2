// shm.h -- POSIX shared-memory byte rings between host ranks of one machine.
//
// One ring per ordered pair (sender creates, receiver opens and removes the name, so
// that nothing is left in /dev/shm once both sides are attached).  Single producer,
// single consumer, head/tail counters with release/acquire ordering.  The host
// collectives use these instead of loopback TCP between ranks of one host (role of
// flagcx/service/shmutils.cc and the shared-memory transport of the FlagCX project).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <string>

#include "flagcx.h"

namespace fcx {

class ShmRing {
 public:
  ShmRing() = default;
  ~ShmRing() { close(); }
  ShmRing(const ShmRing &) = delete;
  ShmRing &operator=(const ShmRing &) = delete;

  // Sender side.  capacity: power of two.  Reserves the pages (fails cleanly when
  // /dev/shm is too small instead of faulting later).
  flagcxResult_t create(const std::string &name, size_t capacity);
  // Receiver side: maps an existing ring and removes its name.
  flagcxResult_t open(const std::string &name);
  void close();
  bool attached() const { return hdr_ != nullptr; }

  // Non-blocking: move up to n bytes, return how many were moved.
  size_t write(const void *src, size_t n);
  size_t read(void *dst, size_t n);

 private:
  struct Header {
    alignas(64) std::atomic<uint64_t> head; // bytes written so far
    alignas(64) std::atomic<uint64_t> tail; // bytes read so far
    alignas(64) uint64_t magic;
    uint64_t capacity;
  };
  Header *hdr_ = nullptr;
  char *data_ = nullptr;
  size_t mapBytes_ = 0;
  std::string name_; // non-empty while this object still owns the name
};

// True when /proc says the process is gone (or a zombie).
bool processIsDead(int pid);

} // namespace fcx
