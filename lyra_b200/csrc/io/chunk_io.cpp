// Parallel whole-file reads and writes for checkpoint chunks: a small thread pool issuing
// pwrite/pread in 8 MiB slices. One chunk file per array shard; every rank calls this for the
// chunks it owns, so a checkpoint streams at the file system's aggregate bandwidth.
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <fcntl.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

constexpr long long kSlice = 8ll << 20;

bool write_all(const char* path, const uint8_t* p, long long n) {
  int fd = ::open(path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return false;
  long long off = 0;
  while (off < n) {
    long long want = n - off < kSlice ? n - off : kSlice;
    ssize_t w = ::pwrite(fd, p + off, (size_t)want, off);
    if (w < 0) {
      if (errno == EINTR) continue;
      ::close(fd);
      return false;
    }
    off += w;
  }
  bool ok = ::fsync(fd) == 0;
  return (::close(fd) == 0) && ok;
}

bool read_all(const char* path, uint8_t* p, long long n) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return false;
  struct stat st;
  if (::fstat(fd, &st) != 0 || st.st_size != n) {
    ::close(fd);
    return false;
  }
  long long off = 0;
  while (off < n) {
    long long want = n - off < kSlice ? n - off : kSlice;
    ssize_t r = ::pread(fd, p + off, (size_t)want, off);
    if (r < 0) {
      if (errno == EINTR) continue;
      ::close(fd);
      return false;
    }
    if (r == 0) break;
    off += r;
  }
  ::close(fd);
  return off == n;
}

template <class Fn>
int run_pool(int n, int threads, Fn fn) {
  std::atomic<int> next{0};
  std::atomic<int> failed{0};  // 1-based index of the first failing item
  if (threads < 1) threads = 1;
  if (threads > n) threads = n;
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    pool.emplace_back([&] {
      for (;;) {
        int i = next.fetch_add(1);
        if (i >= n) return;
        if (!fn(i)) {
          int expected = 0;
          failed.compare_exchange_strong(expected, i + 1);
        }
      }
    });
  }
  for (auto& th : pool) th.join();
  return failed.load();
}

}  // namespace

extern "C" int lyra_io_write_files(int n, const char** paths, const void** ptrs, const long long* sizes, int threads) {
  return run_pool(n, threads, [&](int i) { return write_all(paths[i], static_cast<const uint8_t*>(ptrs[i]), sizes[i]); });
}

extern "C" int lyra_io_read_files(int n, const char** paths, void** ptrs, const long long* sizes, int threads) {
  return run_pool(n, threads, [&](int i) { return read_all(paths[i], static_cast<uint8_t*>(ptrs[i]), sizes[i]); });
}
