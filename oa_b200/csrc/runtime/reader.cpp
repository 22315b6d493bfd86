// Asynchronous file reader: positioned reads submitted to a bounded queue and carried out by worker threads, with
// completions collected in bulk.  Destinations are caller-owned, typically slices of a pinned host buffer that the
// upload stream then copies to the device, so a dataset shard goes file -> pinned memory -> HBM without a bounce.
//
// Parity: Source/Public/Oa/Data/IoUringReader.h (SubmitRead / WaitCompletions / FileSize / IsValid with a queue
// depth).  The reference drives an io_uring; a small pread pool gives the same overlap without a kernel-version
// dependency and keeps page-cache reads at memory speed.
#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

struct Request { void* dst; int64_t offset, bytes; };

struct Reader {
  int fd = -1;
  int64_t size = 0;
  int depth = 32;
  std::mutex m;
  std::condition_variable work, done;
  std::deque<Request> queue;
  int in_flight = 0;          // submitted, not yet collected by WaitCompletions
  int completed = 0;          // finished, not yet collected
  int failed = 0;             // among completed: short or failed reads
  int64_t bytes_read = 0;
  bool stopping = false;
  std::vector<std::thread> workers;
};

static void reader_worker(Reader* r) {
  for (;;) {
    Request q;
    {
      std::unique_lock<std::mutex> lk(r->m);
      r->work.wait(lk, [&] { return r->stopping || !r->queue.empty(); });
      if (r->queue.empty()) return;
      q = r->queue.front();
      r->queue.pop_front();
    }
    int64_t got = 0;
    bool ok = true;
    while (got < q.bytes) {
      ssize_t n = pread(r->fd, static_cast<char*>(q.dst) + got, (size_t)(q.bytes - got), (off_t)(q.offset + got));
      if (n < 0 && errno == EINTR) continue;
      if (n <= 0) { ok = false; break; }
      got += n;
    }
    {
      std::lock_guard<std::mutex> lk(r->m);
      ++r->completed;
      if (!ok) ++r->failed;
      r->bytes_read += got;
    }
    r->done.notify_all();
  }
}

}  // namespace

extern "C" {

void* oa_reader_open(const char* path, int queue_depth, int threads) {
  int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); return nullptr; }
  auto* r = new Reader();
  r->fd = fd; r->size = (int64_t)st.st_size; r->depth = queue_depth > 0 ? queue_depth : 32;
  if (threads <= 0) threads = r->depth < 4 ? r->depth : 4;
  for (int i = 0; i < threads; ++i) r->workers.emplace_back(reader_worker, r);
  return r;
}
void oa_reader_close(void* h) {
  auto* r = static_cast<Reader*>(h);
  if (!r) return;
  { std::lock_guard<std::mutex> lk(r->m); r->stopping = true; }
  r->work.notify_all();
  for (auto& t : r->workers) t.join();
  close(r->fd);
  delete r;
}
int64_t oa_reader_file_size(void* h) { return static_cast<Reader*>(h)->size; }
int64_t oa_reader_bytes_read(void* h) { auto* r = static_cast<Reader*>(h); std::lock_guard<std::mutex> lk(r->m); return r->bytes_read; }
int oa_reader_in_flight(void* h) { auto* r = static_cast<Reader*>(h); std::lock_guard<std::mutex> lk(r->m); return r->in_flight; }

// 0 ok, -1 bad range, -2 queue full (collect completions first)
int oa_reader_submit(void* h, void* dst, int64_t offset, int64_t bytes) {
  auto* r = static_cast<Reader*>(h);
  if (!dst || offset < 0 || bytes < 0 || offset + bytes > r->size) return -1;
  {
    std::lock_guard<std::mutex> lk(r->m);
    if (r->in_flight >= r->depth) return -2;
    ++r->in_flight;
    r->queue.push_back({dst, offset, bytes});
  }
  r->work.notify_one();
  return 0;
}
// Blocks until at least min_complete reads (capped at what is in flight) have finished; collects every finished
// read and returns how many, negated if any of them failed or came back short.
int oa_reader_wait(void* h, int min_complete) {
  auto* r = static_cast<Reader*>(h);
  std::unique_lock<std::mutex> lk(r->m);
  if (min_complete > r->in_flight) min_complete = r->in_flight;
  r->done.wait(lk, [&] { return r->completed >= min_complete; });
  int n = r->completed, bad = r->failed;
  r->in_flight -= n; r->completed = 0; r->failed = 0;
  return bad ? -n : n;
}

}  // extern "C"
