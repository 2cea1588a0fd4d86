// ShmLine: a two-slot shared-memory line for small frames between two processes on one host (the
// leader's per-step pick / control frames).  Slot = sequence parity; the writer publishes with a
// seqlock (odd = being written), the reader re-reads the sequence after copying and reports a torn
// read instead of returning mixed bytes; an ack word lets the writer refuse to lap the reader.
//
// Parity: crates/saber-hip/src/shmline.rs:1-50, :272-411 (post / take_with / exchange, the
// `control_one_slot` + `post_unchecked` pair that reproduces the torn-read hazard in tests).
#include <atomic>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <fcntl.h>
#include <unistd.h>
#include <time.h>

namespace {
constexpr size_t kFrame = 4096;
struct Slot {
  std::atomic<uint64_t> seq;      // 2 * n + 1 while frame n is being written, 2 * n + 2 when complete
  uint32_t len;
  uint8_t data[kFrame];
};
struct Line {
  std::atomic<uint64_t> posted;   // frames published so far
  std::atomic<uint64_t> acked;    // frames the reader has taken
  Slot slot[2];
};
struct Handle { Line* line; int fd; bool owner; char name[128]; int slots; };
uint64_t now_ns() { timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return uint64_t(t.tv_sec) * 1000000000ull + t.tv_nsec; }
}  // namespace

extern "C" {

void* saber_shmline_open(const char* name, int create, int one_slot_control) {
  int fd = shm_open(name, create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) return nullptr;
  if (create && ftruncate(fd, sizeof(Line)) != 0) { close(fd); return nullptr; }
  void* p = mmap(nullptr, sizeof(Line), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) { close(fd); return nullptr; }
  auto* h = new Handle{static_cast<Line*>(p), fd, create != 0, {0}, one_slot_control ? 1 : 2};
  strncpy(h->name, name, sizeof(h->name) - 1);
  if (create) memset(p, 0, sizeof(Line));
  return h;
}

// Publishes frame n = posted. checked = 1 refuses (returns -2) when the reader has not yet taken
// frame n - slots (the slot still holds unread bytes). Returns the frame number or < 0.
int64_t saber_shmline_post(void* hv, const void* data, uint32_t len, int checked) {
  auto* h = static_cast<Handle*>(hv);
  if (len > kFrame) return -1;
  Line* L = h->line;
  const uint64_t n = L->posted.load(std::memory_order_relaxed);
  if (checked && n >= L->acked.load(std::memory_order_acquire) + h->slots) return -2;
  Slot& s = L->slot[n % h->slots];
  s.seq.store(2 * n + 1, std::memory_order_release);
  std::atomic_thread_fence(std::memory_order_release);
  s.len = len;
  memcpy(s.data, data, len);
  std::atomic_thread_fence(std::memory_order_release);
  s.seq.store(2 * n + 2, std::memory_order_release);
  L->posted.store(n + 1, std::memory_order_release);
  return static_cast<int64_t>(n);
}

// Takes frame n (bounded wait). Returns the length, -1 on timeout, -3 when the read was torn
// (the slot was rewritten while it was being copied).
int32_t saber_shmline_take(void* hv, uint64_t n, void* out, uint32_t cap, uint64_t timeout_ns) {
  auto* h = static_cast<Handle*>(hv);
  Line* L = h->line;
  Slot& s = L->slot[n % h->slots];
  const uint64_t t0 = now_ns();
  while (s.seq.load(std::memory_order_acquire) < 2 * n + 2) {
    if (now_ns() - t0 > timeout_ns) return -1;
  }
  const uint64_t before = s.seq.load(std::memory_order_acquire);
  if (before != 2 * n + 2) return -3;
  const uint32_t len = s.len;
  if (len > cap) return -1;
  memcpy(out, s.data, len);
  std::atomic_thread_fence(std::memory_order_acquire);
  if (s.seq.load(std::memory_order_acquire) != before) return -3;
  L->acked.store(n + 1, std::memory_order_release);
  return static_cast<int32_t>(len);
}

uint64_t saber_shmline_posted(void* hv) { return static_cast<Handle*>(hv)->line->posted.load(); }

void saber_shmline_close(void* hv) {
  auto* h = static_cast<Handle*>(hv);
  munmap(h->line, sizeof(Line));
  close(h->fd);
  if (h->owner) shm_unlink(h->name);
  delete h;
}

}  // extern "C"
