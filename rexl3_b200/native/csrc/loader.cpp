// Parallel file-range reader for pack loading: many (offset, size) ranges of one file are cut into chunks and read by a pool of
// threads straight into caller-provided destinations (e.g. slices of one pinned staging buffer), optionally with O_DIRECT through
// per-thread aligned bounce buffers so a 100 GB pack does not churn the page cache.  Role of the reference's pipelined weight loader
// (crates/cuda/src/loader.rs: O_DIRECT, staged, multi-thread); the host->device copies are issued by the caller from the filled buffer.
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int64_t CHUNK = 8 << 20;
constexpr int64_t ALIGN = 4096;

struct Job {
  int64_t off, size;
  char* dst;
};

// read [off, off+size) into dst; returns 0 or an errno value (EIO for a short file)
int read_plain(int fd, int64_t off, int64_t size, char* dst) {
  while (size > 0) {
    const ssize_t r = pread(fd, dst, (size_t)size, (off_t)off);
    if (r < 0) {
      if (errno == EINTR) continue;
      return errno;
    }
    if (r == 0) return EIO;
    off += r, dst += r, size -= r;
  }
  return 0;
}

int read_direct(int fd, int64_t off, int64_t size, char* dst, char* bounce, int64_t file_size) {
  const int64_t a0 = off / ALIGN * ALIGN;
  const int64_t a1 = std::min((off + size + ALIGN - 1) / ALIGN * ALIGN, (file_size + ALIGN - 1) / ALIGN * ALIGN);
  int64_t got = 0;
  while (a0 + got < a1) {
    const ssize_t r = pread(fd, bounce + got, (size_t)(a1 - a0 - got), (off_t)(a0 + got));
    if (r < 0) {
      if (errno == EINTR) continue;
      return errno;
    }
    if (r == 0) break;               // end of file inside the last aligned block
    got += r;
  }
  if (a0 + got < off + size) return EIO;
  std::memcpy(dst, bounce + (off - a0), (size_t)size);
  return 0;
}

}  // namespace

extern "C" {

// Returns 0, or an errno value (the first failure).  `direct` != 0 asks for O_DIRECT; if the file system refuses it the read falls
// back to buffered I/O and *used_direct (may be null) reports 0.
int rx_read_ranges(const char* path, int n, const int64_t* offsets, const int64_t* sizes, void* const* dsts, int threads, int direct,
                   int* used_direct) {
  if (n < 0) return EINVAL;
  int fd = -1;
  if (direct) fd = open(path, O_RDONLY | O_DIRECT);
  const bool is_direct = fd >= 0;
  if (fd < 0) fd = open(path, O_RDONLY);
  if (fd < 0) return errno;
  if (used_direct) *used_direct = is_direct ? 1 : 0;
  const int64_t file_size = (int64_t)lseek(fd, 0, SEEK_END);
  std::vector<Job> jobs;
  for (int i = 0; i < n; ++i) {
    if (offsets[i] < 0 || sizes[i] < 0 || offsets[i] + sizes[i] > file_size) {
      close(fd);
      return EIO;
    }
    for (int64_t o = 0; o < sizes[i]; o += CHUNK) jobs.push_back({offsets[i] + o, std::min(CHUNK, sizes[i] - o), (char*)dsts[i] + o});
  }
  std::atomic<size_t> next(0);
  std::atomic<int> err(0);
  int nt = threads > 0 ? threads : 8;
  nt = std::max(1, std::min<int>(nt, (int)std::max<size_t>(jobs.size(), 1)));
  auto work = [&]() {
    char* bounce = nullptr;
    if (is_direct && posix_memalign((void**)&bounce, ALIGN, (size_t)(CHUNK + 2 * ALIGN)) != 0) {
      err.store(ENOMEM);
      return;
    }
    for (;;) {
      const size_t j = next.fetch_add(1);
      if (j >= jobs.size() || err.load() != 0) break;
      const Job& jb = jobs[j];
      const int e = is_direct ? read_direct(fd, jb.off, jb.size, jb.dst, bounce, file_size) : read_plain(fd, jb.off, jb.size, jb.dst);
      if (e != 0) {
        int zero = 0;
        err.compare_exchange_strong(zero, e);
      }
    }
    std::free(bounce);
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < nt; ++i) pool.emplace_back(work);
  work();
  for (auto& th : pool) th.join();
  close(fd);
  return err.load();
}

}  // extern "C"
