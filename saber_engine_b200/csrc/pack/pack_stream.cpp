// Streaming pack loader: O_DIRECT reads in chunk-sized pieces through a small ring of pinned
// staging buffers, SHA-256 of every chunk checked BEFORE the bytes are sent to the device, then an
// asynchronous host-to-device copy.  Nothing unverified ever reaches device memory.
//
// Parity: crates/saber-mem/src/pack/stream.rs (PackStream: O_DIRECT, 4 MiB chunk digests) and
// crates/saber-mem/src/upload.rs:1-40 (pinned staging ring, sha256 before H2D).
#include <cuda_runtime.h>
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <vector>

namespace {

struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  static constexpr uint32_t K[64] = {
      0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
      0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
      0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
      0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
      0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
      0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
      0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
      0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      const uint32_t ch = (e & f) ^ (~e & g);
      const uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      const uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    len += n;
    if (fill) {
      const size_t take = n < 64 - fill ? n : 64 - fill;
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
    while (n >= 64) { block(p); p += 64; n -= 64; }
    if (n) { memcpy(buf, p, n); fill = n; }
  }
  void final(uint8_t out[32]) {
    const uint64_t bits = len * 8;
    uint8_t pad[72] = {0x80};
    const size_t padlen = (fill < 56) ? 56 - fill : 120 - fill;
    update(pad, padlen);
    uint8_t lb[8];
    for (int i = 0; i < 8; ++i) lb[i] = uint8_t(bits >> (56 - 8 * i));
    update(lb, 8);
    for (int i = 0; i < 8; ++i) { out[4 * i] = h[i] >> 24; out[4 * i + 1] = h[i] >> 16; out[4 * i + 2] = h[i] >> 8; out[4 * i + 3] = h[i]; }
  }
};
constexpr uint32_t Sha256::K[64];

struct Stream {
  int fd = -1;
  bool direct = false;
  size_t chunk = 0;
  std::vector<void*> ring;      // pinned (or plain aligned) staging buffers
  std::vector<cudaEvent_t> done;
  bool pinned = false;
  uint64_t bytes_read = 0, chunks_verified = 0;
};

}  // namespace

extern "C" {

void saber_sha256(const void* data, size_t n, void* out32) {
  Sha256 s;
  s.update(static_cast<const uint8_t*>(data), n);
  s.final(static_cast<uint8_t*>(out32));
}

// ring_slots staging buffers of chunk_bytes each; use_cuda = 0 keeps everything on the host (tests).
void* saber_pack_stream_open(const char* path, size_t chunk_bytes, int ring_slots, int use_cuda) {
  auto* s = new Stream();
  s->fd = open(path, O_RDONLY | O_DIRECT);
  s->direct = s->fd >= 0;
  if (s->fd < 0) s->fd = open(path, O_RDONLY);       // file systems without O_DIRECT (tmpfs)
  if (s->fd < 0) { delete s; return nullptr; }
  s->chunk = chunk_bytes;
  for (int i = 0; i < ring_slots; ++i) {
    void* p = nullptr;
    if (use_cuda && cudaHostAlloc(&p, chunk_bytes, cudaHostAllocDefault) == cudaSuccess) {
      s->pinned = true;
    } else if (posix_memalign(&p, 4096, chunk_bytes) != 0) {
      p = nullptr;
    }
    if (!p) break;
    s->ring.push_back(p);
    cudaEvent_t e = nullptr;
    if (use_cuda) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    s->done.push_back(e);
  }
  if (s->ring.empty()) { close(s->fd); delete s; return nullptr; }
  return s;
}

int saber_pack_stream_is_direct(void* h) { return static_cast<Stream*>(h)->direct ? 1 : 0; }

// Streams [data_off, data_off + length) to dst (device memory when stream_or_null != 0 / to_device,
// host memory otherwise), verifying chunk j against digests[32 * j].  data_off is 4096-aligned by
// the format.  Returns 0, -1 on a read error, or 1 + j for the first chunk whose digest is wrong.
int saber_pack_stream_record(void* h, uint64_t data_off, uint64_t length, void* dst, int to_device,
                             const uint8_t* digests, cudaStream_t stream) {
  auto* s = static_cast<Stream*>(h);
  const size_t n_chunks = (length + s->chunk - 1) / s->chunk;
  for (size_t j = 0; j < n_chunks; ++j) {
    const size_t slot = j % s->ring.size();
    if (to_device && s->done[slot] && j >= s->ring.size()) cudaEventSynchronize(s->done[slot]);
    const uint64_t off = data_off + j * s->chunk;
    const size_t want = static_cast<size_t>(length - j * s->chunk < s->chunk ? length - j * s->chunk : s->chunk);
    const size_t rd = s->direct ? ((want + 4095) / 4096) * 4096 : want;   // O_DIRECT: whole sectors
    size_t got = 0;
    while (got < want) {
      const ssize_t r = pread(s->fd, static_cast<uint8_t*>(s->ring[slot]) + got, rd - got, off + got);
      if (r < 0) { if (errno == EINTR) continue; return -1; }
      if (r == 0) break;
      got += static_cast<size_t>(r);
    }
    if (got < want) return -1;
    s->bytes_read += want;
    if (digests) {
      uint8_t d[32];
      saber_sha256(s->ring[slot], want, d);
      if (memcmp(d, digests + 32 * j, 32) != 0) return 1 + static_cast<int>(j);
      ++s->chunks_verified;
    }
    uint8_t* out = static_cast<uint8_t*>(dst) + j * s->chunk;
    if (to_device) {
      if (cudaMemcpyAsync(out, s->ring[slot], want, cudaMemcpyHostToDevice, stream) != cudaSuccess) return -1;
      if (s->done[slot]) cudaEventRecord(s->done[slot], stream);
    } else {
      memcpy(out, s->ring[slot], want);
    }
  }
  if (to_device) cudaStreamSynchronize(stream);
  return 0;
}

uint64_t saber_pack_stream_bytes(void* h) { return static_cast<Stream*>(h)->bytes_read; }
uint64_t saber_pack_stream_verified(void* h) { return static_cast<Stream*>(h)->chunks_verified; }

void saber_pack_stream_close(void* h) {
  auto* s = static_cast<Stream*>(h);
  if (!s) return;
  for (size_t i = 0; i < s->ring.size(); ++i) {
    if (s->pinned) cudaFreeHost(s->ring[i]); else free(s->ring[i]);
    if (s->done[i]) cudaEventDestroy(s->done[i]);
  }
  close(s->fd);
  delete s;
}

}  // extern "C"
