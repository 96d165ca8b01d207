#include "xpool/shmem.hpp"

#include <errno.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace xpool {

SharedMemory::~SharedMemory() { close(); }

int SharedMemory::create(const std::string& name, size_t bytes) {
  close();
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) return -errno;
  if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    int e = errno;
    ::close(fd);
    shm_unlink(name.c_str());
    return -e;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  int e = errno;
  ::close(fd);
  if (p == MAP_FAILED) {
    shm_unlink(name.c_str());
    return -e;
  }
  name_ = name;
  data_ = p;
  size_ = bytes;
  owner_ = true;
  return 0;
}

int SharedMemory::attach(const std::string& name) {
  close();
  int fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) return -errno;
  struct stat st;
  if (fstat(fd, &st) != 0) {
    int e = errno;
    ::close(fd);
    return -e;
  }
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  int e = errno;
  ::close(fd);
  if (p == MAP_FAILED) return -e;
  name_ = name;
  data_ = p;
  size_ = static_cast<size_t>(st.st_size);
  owner_ = false;
  return 0;
}

void SharedMemory::close() {
  if (data_ != nullptr) {
    munmap(data_, size_);
    if (owner_) shm_unlink(name_.c_str());
  }
  data_ = nullptr;
  size_ = 0;
  owner_ = false;
  name_.clear();
}

}  // namespace xpool
