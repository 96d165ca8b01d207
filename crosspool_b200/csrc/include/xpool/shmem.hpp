// POSIX shared-memory region: the owner creates it exclusively with mode 0600
// and unlinks it on destruction; attachers map an existing name. Used by the
// ECS control channel and by the CPU loopback fabric. (Reference counterpart:
// src/cext-include/xpool/utils/shmem.hpp, src/cext/utils/shmem.cpp.)
#pragma once

#include <stddef.h>
#include <stdint.h>

#include <string>

namespace xpool {

class SharedMemory {
 public:
  SharedMemory() = default;
  ~SharedMemory();
  SharedMemory(const SharedMemory&) = delete;
  SharedMemory& operator=(const SharedMemory&) = delete;

  // Returns 0 or -errno.
  int create(const std::string& name, size_t bytes);
  int attach(const std::string& name);
  void close();

  void* data() const { return data_; }
  size_t size() const { return size_; }
  bool owner() const { return owner_; }
  const std::string& name() const { return name_; }

 private:
  std::string name_;
  void* data_ = nullptr;
  size_t size_ = 0;
  bool owner_ = false;
};

}  // namespace xpool
