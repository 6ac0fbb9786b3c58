// Token-block source and prefetch pool (the native counterpart of the reference's Grain
// DataLoader workers, lyra/data.py:78-94).
//
// A token source is either a set of ArrayRecord shards (one record per document chunk of
// little-endian int32 tokens, concatenated across records and shards) or a raw int32 region of a
// file (the payload of a .npy). Block i of size S is tokens [i*S, i*S + S] (S + 1 tokens: inputs and
// the one-token-shifted labels, lyra/data.py:64-67). The pool fills caller-owned (pinned) buffers
// asynchronously; the Python side decides the block order and owns the resumable sampler state.
#include <algorithm>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <fcntl.h>
#include <map>
#include <mutex>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

extern "C" {
void* lyra_ar_reader_open(const char* path);
long long lyra_ar_reader_num_records(void* handle);
long long lyra_ar_reader_record_size(void* handle, long long idx);
long long lyra_ar_reader_read(void* handle, long long idx, long long offset, long long n, void* out);
void lyra_ar_reader_close(void* handle);
}

namespace {

struct TokenSource {
  // ArrayRecord mode
  std::vector<std::string> shards;
  std::vector<long long> shard_first_record;  // global record index of each shard's first record
  std::vector<long long> record_offset;       // token offset of each global record, plus the total at the end
  // raw mode
  const int32_t* raw = nullptr;
  void* raw_map = nullptr;
  size_t raw_map_size = 0;
  long long total = 0;

  struct Readers {
    std::vector<void*> handles;
    ~Readers() {
      for (void* h : handles)
        if (h) lyra_ar_reader_close(h);
    }
  };

  bool read(Readers& rd, long long start, long long count, int32_t* out) const {
    if (start < 0 || start + count > total) return false;
    if (raw) {
      memcpy(out, raw + start, size_t(count) * 4);
      return true;
    }
    if (rd.handles.empty()) rd.handles.assign(shards.size(), nullptr);
    long long rec = (long long)(std::upper_bound(record_offset.begin(), record_offset.end(), start) - record_offset.begin()) - 1;
    while (count > 0) {
      const long long local = start - record_offset[rec];
      const long long take = std::min(count, record_offset[rec + 1] - start);
      const size_t shard = size_t(std::upper_bound(shard_first_record.begin(), shard_first_record.end(), rec) - shard_first_record.begin()) - 1;
      if (!rd.handles[shard]) rd.handles[shard] = lyra_ar_reader_open(shards[shard].c_str());
      if (!rd.handles[shard]) return false;
      if (take > 0 &&
          lyra_ar_reader_read(rd.handles[shard], rec - shard_first_record[shard], local * 4, take * 4, out) != take * 4)
        return false;
      out += take;
      start += take;
      count -= take;
      ++rec;
    }
    return true;
  }
};

struct Job {
  int ticket;
  long long block;
  int32_t* out;
};

struct Loader {
  const TokenSource* src;
  long long block_tokens;
  std::vector<std::thread> threads;
  std::mutex mu;
  std::condition_variable cv_jobs, cv_done;
  std::deque<Job> jobs;
  std::map<int, int> done;  // ticket -> status (0 ok, -1 failed)
  int next_ticket = 0;
  bool stop = false;

  void worker() {
    TokenSource::Readers readers;
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_jobs.wait(lk, [&] { return stop || !jobs.empty(); });
        if (stop && jobs.empty()) return;
        job = jobs.front();
        jobs.pop_front();
      }
      const bool ok = src->read(readers, job.block * block_tokens, block_tokens + 1, job.out);
      {
        std::lock_guard<std::mutex> lk(mu);
        done[job.ticket] = ok ? 0 : -1;
      }
      cv_done.notify_all();
    }
  }
};

}  // namespace

extern "C" {

void* lyra_tokens_open(int n_shards, const char** paths) {
  TokenSource* s = new TokenSource;
  s->record_offset.push_back(0);
  long long records = 0;
  for (int i = 0; i < n_shards; ++i) {
    void* r = lyra_ar_reader_open(paths[i]);
    if (!r) {
      delete s;
      return nullptr;
    }
    s->shards.emplace_back(paths[i]);
    s->shard_first_record.push_back(records);
    const long long n = lyra_ar_reader_num_records(r);
    for (long long j = 0; j < n; ++j) {
      const long long bytes = lyra_ar_reader_record_size(r, j);
      if (bytes < 0 || bytes % 4) {
        lyra_ar_reader_close(r);
        delete s;
        return nullptr;
      }
      s->record_offset.push_back(s->record_offset.back() + bytes / 4);
    }
    records += n;
    lyra_ar_reader_close(r);
  }
  s->total = s->record_offset.back();
  return s;
}

void* lyra_tokens_open_raw(const char* path, long long byte_offset, long long n_tokens) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < byte_offset + n_tokens * 4) {
    ::close(fd);
    return nullptr;
  }
  void* m = mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) return nullptr;
  TokenSource* s = new TokenSource;
  s->raw_map = m;
  s->raw_map_size = size_t(st.st_size);
  s->raw = reinterpret_cast<const int32_t*>(static_cast<const uint8_t*>(m) + byte_offset);
  s->total = n_tokens;
  return s;
}

long long lyra_tokens_count(void* handle) { return static_cast<TokenSource*>(handle)->total; }

long long lyra_tokens_num_records(void* handle) {
  TokenSource* s = static_cast<TokenSource*>(handle);
  return s->raw ? 1 : (long long)s->record_offset.size() - 1;
}

int lyra_tokens_read(void* handle, long long start, long long count, int32_t* out) {
  TokenSource::Readers readers;
  return static_cast<TokenSource*>(handle)->read(readers, start, count, out) ? 0 : -1;
}

void lyra_tokens_close(void* handle) {
  TokenSource* s = static_cast<TokenSource*>(handle);
  if (s->raw_map) munmap(s->raw_map, s->raw_map_size);
  delete s;
}

void* lyra_loader_create(void* src, long long block_tokens, int threads) {
  Loader* l = new Loader;
  l->src = static_cast<TokenSource*>(src);
  l->block_tokens = block_tokens;
  for (int i = 0; i < std::max(threads, 1); ++i) l->threads.emplace_back([l] { l->worker(); });
  return l;
}

int lyra_loader_submit(void* handle, long long block, int32_t* out) {
  Loader* l = static_cast<Loader*>(handle);
  int ticket;
  {
    std::lock_guard<std::mutex> lk(l->mu);
    ticket = l->next_ticket++;
    l->jobs.push_back({ticket, block, out});
  }
  l->cv_jobs.notify_one();
  return ticket;
}

int lyra_loader_wait(void* handle, int ticket) {
  Loader* l = static_cast<Loader*>(handle);
  std::unique_lock<std::mutex> lk(l->mu);
  l->cv_done.wait(lk, [&] { return l->done.count(ticket) > 0; });
  const int status = l->done[ticket];
  l->done.erase(ticket);
  return status;
}

void lyra_loader_destroy(void* handle) {
  Loader* l = static_cast<Loader*>(handle);
  {
    std::lock_guard<std::mutex> lk(l->mu);
    l->stop = true;
  }
  l->cv_jobs.notify_all();
  for (auto& t : l->threads) t.join();
  delete l;
}

}  // extern "C"
