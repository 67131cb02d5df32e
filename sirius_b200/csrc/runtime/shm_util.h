// POSIX shared-memory helpers for the host-side runtime: a named segment holding one fixed-layout
// struct, process-shared mutex / condition variable wrappers with monotonic timed waits.
// (The reference uses Boost.Interprocess managed segments, common/inf_tra_comm/bip_helper.h; the
// layouts here are plain structs, so the byte format is this library's own.)
#pragma once
#include <errno.h>
#include <fcntl.h>
#include <pthread.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <string>

namespace srt {
namespace shm {

struct Mutex {
  pthread_mutex_t m;
  void init() {
    pthread_mutexattr_t a;
    pthread_mutexattr_init(&a);
    pthread_mutexattr_setpshared(&a, PTHREAD_PROCESS_SHARED);
    pthread_mutexattr_setrobust(&a, PTHREAD_MUTEX_ROBUST);
    pthread_mutex_init(&m, &a);
    pthread_mutexattr_destroy(&a);
  }
  void lock() {
    int r = pthread_mutex_lock(&m);
    if (r == EOWNERDEAD) pthread_mutex_consistent(&m);  // previous owner died: state is plain data
  }
  void unlock() { pthread_mutex_unlock(&m); }
};

struct Cond {
  pthread_cond_t c;
  void init() {
    pthread_condattr_t a;
    pthread_condattr_init(&a);
    pthread_condattr_setpshared(&a, PTHREAD_PROCESS_SHARED);
    pthread_condattr_setclock(&a, CLOCK_MONOTONIC);
    pthread_cond_init(&c, &a);
    pthread_condattr_destroy(&a);
  }
  void wait(Mutex& m) {
    int r = pthread_cond_wait(&c, &m.m);
    if (r == EOWNERDEAD) pthread_mutex_consistent(&m.m);
  }
  // returns false on timeout
  bool wait_until(Mutex& m, const timespec& deadline) {
    int r = pthread_cond_timedwait(&c, &m.m, &deadline);
    if (r == EOWNERDEAD) pthread_mutex_consistent(&m.m);
    return r != ETIMEDOUT;
  }
  void notify_one() { pthread_cond_signal(&c); }
  void notify_all() { pthread_cond_broadcast(&c); }
};

struct Guard {
  Mutex& m;
  explicit Guard(Mutex& mm) : m(mm) { m.lock(); }
  ~Guard() { m.unlock(); }
};

inline timespec deadline_after_ms(int64_t ms) {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  ts.tv_sec += ms / 1000;
  ts.tv_nsec += (ms % 1000) * 1000000;
  if (ts.tv_nsec >= 1000000000) { ts.tv_sec += 1; ts.tv_nsec -= 1000000000; }
  return ts;
}

// Header every segment starts with; `ready` is published last by the creator.
struct SegHeader {
  uint32_t magic;
  uint32_t bytes;
  std::atomic<int> ready;
  // Who made this incarnation of the segment. A segment outlives a creator that crashed or was killed, and a
  // process of the next job that opens the name before the new creator has replaced it would map the orphan
  // (and then run on different barriers and ledgers than its peers). Openers therefore only accept a segment
  // whose creator is alive: the creator always unlinks and recreates the name when it starts, so an orphan is
  // by definition one whose creator is gone.
  int32_t owner_pid;
  uint64_t owner_start;  // the creator's start time (clock ticks since boot, /proc/<pid>/stat field 22): pids are reused
};

// Start time of a process in clock ticks since boot, 0 if it cannot be read.
inline uint64_t process_start_ticks(int pid) {
  char path[64], buf[1024];
  snprintf(path, sizeof(path), "/proc/%d/stat", pid);
  int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return 0;
  ssize_t n = ::read(fd, buf, sizeof(buf) - 1);
  ::close(fd);
  if (n <= 0) return 0;
  buf[n] = 0;
  const char* p = strrchr(buf, ')');  // the command name may contain spaces and parentheses
  if (!p) return 0;
  int field = 2;
  for (++p; *p; ++p) {
    if (*p != ' ') continue;
    if (++field == 22) return strtoull(p + 1, nullptr, 10);
  }
  return 0;
}

inline bool owner_alive(const SegHeader& h) {
  if (h.owner_pid <= 0) return false;
  if (kill(h.owner_pid, 0) != 0 && errno == ESRCH) return false;
  const uint64_t st = process_start_ticks(h.owner_pid);
  return st == 0 || h.owner_start == 0 || st == h.owner_start;  // unreadable /proc: the pid check has to do
}

// Maps a named segment holding a T (T begins with a SegHeader named `hdr`). The creator
// zero-fills it and runs init(T*) before publishing; openers wait up to timeout_ms for it.
template <typename T>
class Segment {
 public:
  Segment() = default;
  ~Segment() { close(); }
  Segment(const Segment&) = delete;
  Segment& operator=(const Segment&) = delete;

  template <typename Init>
  bool create(const std::string& name, uint32_t magic, bool remove_existing, Init init, std::string* err) {
    name_ = name[0] == '/' ? name : "/" + name;
    if (remove_existing) shm_unlink(name_.c_str());
    int fd = shm_open(name_.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0) { *err = "shm_open(create) " + name_ + ": " + strerror(errno); return false; }
    if (ftruncate(fd, sizeof(T)) != 0) { *err = std::string("ftruncate: ") + strerror(errno); ::close(fd); return false; }
    void* p = mmap(nullptr, sizeof(T), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) { *err = std::string("mmap: ") + strerror(errno); return false; }
    ptr_ = static_cast<T*>(p);
    owner_ = true;
    if (ptr_->hdr.ready.load(std::memory_order_acquire) == 1 && ptr_->hdr.magic == magic) {  // reuse: now this process vouches for it
      ptr_->hdr.owner_pid = (int32_t)getpid();
      ptr_->hdr.owner_start = process_start_ticks((int)getpid());
      return true;
    }
    memset(p, 0, sizeof(T));
    ptr_->hdr.magic = magic;
    ptr_->hdr.bytes = (uint32_t)sizeof(T);
    ptr_->hdr.owner_pid = (int32_t)getpid();
    ptr_->hdr.owner_start = process_start_ticks((int)getpid());
    init(ptr_);
    ptr_->hdr.ready.store(1, std::memory_order_release);
    return true;
  }

  bool open(const std::string& name, uint32_t magic, int timeout_ms, std::string* err) {
    name_ = name[0] == '/' ? name : "/" + name;
    const timespec dl = deadline_after_ms(timeout_ms);
    for (;;) {
      int fd = shm_open(name_.c_str(), O_RDWR, 0600);
      if (fd >= 0) {
        struct stat st;
        if (fstat(fd, &st) == 0 && (size_t)st.st_size >= sizeof(T)) {
          void* p = mmap(nullptr, sizeof(T), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
          ::close(fd);
          if (p == MAP_FAILED) { *err = std::string("mmap: ") + strerror(errno); return false; }
          ptr_ = static_cast<T*>(p);
          bool orphan = false;
          for (;;) {
            if (ptr_->hdr.ready.load(std::memory_order_acquire) == 1) {
              if (ptr_->hdr.magic != magic || ptr_->hdr.bytes != sizeof(T)) {
                *err = "segment " + name_ + " has a different layout";
                return false;
              }
              if (owner_alive(ptr_->hdr)) return true;
              orphan = true;  // left by a creator that is gone: wait for this job's creator to replace it
              break;
            }
            if (expired(dl)) { *err = "segment " + name_ + " never became ready"; return false; }
            usleep(1000);
          }
          munmap(ptr_, sizeof(T));
          ptr_ = nullptr;
          if (orphan && expired(dl)) {
            *err = "segment " + name_ + " was left by a process that no longer runs, and nobody replaced it";
            return false;
          }
          usleep(2000);
          continue;
        }
        ::close(fd);
      }
      if (expired(dl)) { *err = "segment " + name_ + " does not exist"; return false; }
      usleep(2000);
    }
  }

  void close() {
    if (ptr_) munmap(ptr_, sizeof(T));
    ptr_ = nullptr;
  }
  void unlink() {
    if (!name_.empty()) shm_unlink(name_.c_str());
  }
  T* get() const { return ptr_; }
  bool owner() const { return owner_; }
  const std::string& name() const { return name_; }

 private:
  static bool expired(const timespec& dl) {
    timespec now;
    clock_gettime(CLOCK_MONOTONIC, &now);
    return now.tv_sec > dl.tv_sec || (now.tv_sec == dl.tv_sec && now.tv_nsec >= dl.tv_nsec);
  }
  T* ptr_ = nullptr;
  bool owner_ = false;
  std::string name_;
};

}  // namespace shm
}  // namespace srt
