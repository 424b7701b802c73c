// Host-side native runtime: checkpoint I/O (.fdl), SHA-256, the CPU RNG used by samplers, the
// prefetching batch loader, and the El Che cadence scheduler.
//
// These are the parts the reference implements natively in Rust
// (flodl/src/nn/checkpoint.rs, flodl/src/rng.rs, flodl/src/data/prefetch.rs,
// flodl/src/distributed/el_che.rs); here they are C++17 over the libtorch C++ API, exposed to
// Python through pybind11.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>
#include <zlib.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <optional>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace {

using torch::Tensor;

// ================================================================================== SHA-256
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    std::memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
        0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
        0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
        0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
        0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
        0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
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
  void update(const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    len += n;
    while (n) {
      const size_t take = std::min(n, 64 - fill);
      std::memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  std::array<uint8_t, 32> digest() {
    const uint64_t bits = len * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = uint8_t(bits >> (56 - 8 * i));
    update(lenb, 8);
    std::array<uint8_t, 32> out;
    for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) out[4 * i + j] = uint8_t(h[i] >> (24 - 8 * j));
    return out;
  }
};

std::string sha256_hex(const std::string& data) {
  Sha256 s;
  s.update(data.data(), data.size());
  auto d = s.digest();
  static const char* hex = "0123456789abcdef";
  std::string out(64, '0');
  for (int i = 0; i < 32; ++i) { out[2 * i] = hex[d[i] >> 4]; out[2 * i + 1] = hex[d[i] & 15]; }
  return out;
}

// ============================================================================ .fdl checkpoints
// Layout (little-endian): "FDLC" | u32 version | 32-byte hash | u32 count |
//   count x { u32 name_len, name, u32 ndim, i64 shape[ndim], u8 dtype, u64 nbytes, raw data }
// dtype tags: 1=f16 2=bf16 3=f32 4=f64 5=i32 6=i64. A ".gz" path gzips the whole stream.
struct ByteSink {
  gzFile gz = nullptr;
  FILE* fp = nullptr;
  std::string* mem = nullptr;
  void write(const void* p, size_t n) {
    if (mem) { mem->append(static_cast<const char*>(p), n); return; }
    if (gz) {
      const char* c = static_cast<const char*>(p);
      while (n) {
        const unsigned chunk = static_cast<unsigned>(std::min<size_t>(n, 1u << 30));
        TORCH_CHECK(gzwrite(gz, c, chunk) == (int)chunk, "checkpoint: gzip write failed");
        c += chunk; n -= chunk;
      }
      return;
    }
    TORCH_CHECK(fwrite(p, 1, n, fp) == n, "checkpoint: write failed");
  }
  template <typename T> void put(T v) { write(&v, sizeof(T)); }
};
struct ByteSource {
  gzFile gz = nullptr;
  const std::string* mem = nullptr;
  size_t pos = 0;
  // Bytes that can still be read from an in-memory source (files: unknown, reported as "unbounded").
  uint64_t remaining() const { return mem ? static_cast<uint64_t>(mem->size() - pos) : UINT64_MAX; }
  void read(void* p, size_t n) {
    if (mem) {
      TORCH_CHECK(pos <= mem->size() && n <= mem->size() - pos, "checkpoint: unexpected end of data");
      std::memcpy(p, mem->data() + pos, n);
      pos += n;
      return;
    }
    char* c = static_cast<char*>(p);
    while (n) {
      const unsigned chunk = static_cast<unsigned>(std::min<size_t>(n, 1u << 30));
      TORCH_CHECK(gzread(gz, c, chunk) == (int)chunk, "checkpoint: unexpected end of file");
      c += chunk; n -= chunk;
    }
  }
  // Skip `n` payload bytes without materialising them.
  void skip(uint64_t n) {
    if (mem) {
      TORCH_CHECK(pos <= mem->size() && n <= mem->size() - pos, "checkpoint: unexpected end of data");
      pos += static_cast<size_t>(n);
      return;
    }
    TORCH_CHECK(n <= static_cast<uint64_t>(INT64_MAX) && gzseek(gz, static_cast<z_off_t>(n), SEEK_CUR) >= 0,
                "checkpoint: unexpected end of file");
  }
  template <typename T> T get() { T v; read(&v, sizeof(T)); return v; }
};

uint8_t dtype_tag(at::ScalarType t) {
  switch (t) {
    case at::kHalf: return 1;
    case at::kBFloat16: return 2;
    case at::kFloat: return 3;
    case at::kDouble: return 4;
    case at::kInt: return 5;
    case at::kLong: return 6;
    default: TORCH_CHECK(false, "checkpoint: unsupported dtype ", t);
  }
}
at::ScalarType tag_dtype(uint8_t tag) {
  switch (tag) {
    case 1: return at::kHalf;
    case 2: return at::kBFloat16;
    case 3: return at::kFloat;
    case 4: return at::kDouble;
    case 5: return at::kInt;
    case 6: return at::kLong;
    default: TORCH_CHECK(false, "checkpoint: unknown dtype tag ", (int)tag);
  }
}

void write_tensor_record(ByteSink& s, const Tensor& t_in) {
  Tensor t = t_in.detach().to(torch::kCPU).contiguous();
  s.put<uint32_t>(static_cast<uint32_t>(t.dim()));
  for (int64_t d : t.sizes()) s.put<int64_t>(d);
  s.put<uint8_t>(dtype_tag(t.scalar_type()));
  const uint64_t nbytes = t.numel() * t.element_size();
  s.put<uint64_t>(nbytes);
  if (nbytes) s.write(t.data_ptr(), nbytes);
}
// The header of a record comes from an untrusted file: nothing is allocated until its dimensions are
// non-negative, their product (checked for overflow) times the element size equals the stated byte
// count, and - for in-memory sources - that many bytes are actually there. `skip_payload` moves past
// the data instead of reading it (key listings).
Tensor read_tensor_record(ByteSource& s, bool skip_payload = false) {
  const uint32_t ndim = s.get<uint32_t>();
  TORCH_CHECK(ndim <= 16, "checkpoint: implausible rank ", ndim);
  std::vector<int64_t> shape(ndim);
  uint64_t numel = 1;
  for (auto& d : shape) {
    d = s.get<int64_t>();
    TORCH_CHECK(d >= 0, "checkpoint: negative dimension ", d);
    TORCH_CHECK(d == 0 || numel <= (uint64_t(1) << 56) / static_cast<uint64_t>(d), "checkpoint: tensor size overflows");
    numel *= static_cast<uint64_t>(d);
  }
  const at::ScalarType st = tag_dtype(s.get<uint8_t>());
  const uint64_t nbytes = s.get<uint64_t>();
  TORCH_CHECK(nbytes == numel * c10::elementSize(st), "checkpoint: byte count does not match shape");
  TORCH_CHECK(nbytes <= s.remaining(), "checkpoint: record is longer than the data that follows");
  if (skip_payload) {
    s.skip(nbytes);
    return Tensor();
  }
  Tensor t = torch::empty(shape, torch::dtype(st));
  if (nbytes) s.read(t.data_ptr(), nbytes);
  return t;
}

bool ends_with(const std::string& s, const std::string& suf) {
  return s.size() >= suf.size() && s.compare(s.size() - suf.size(), suf.size(), suf) == 0;
}

void fdl_write_stream(ByteSink& s, const std::vector<std::pair<std::string, Tensor>>& entries, const std::string& hash32,
                      uint32_t version) {
  s.write("FDLC", 4);
  s.put<uint32_t>(version);
  std::string h = hash32;
  h.resize(32, '\0');
  s.write(h.data(), 32);
  s.put<uint32_t>(static_cast<uint32_t>(entries.size()));
  for (auto& e : entries) {
    s.put<uint32_t>(static_cast<uint32_t>(e.first.size()));
    s.write(e.first.data(), e.first.size());
    write_tensor_record(s, e.second);
  }
}

void fdl_save(const std::string& path, const std::vector<std::pair<std::string, Tensor>>& entries, const std::string& hash32,
              uint32_t version) {
  ByteSink s;
  if (ends_with(path, ".gz")) {
    s.gz = gzopen(path.c_str(), "wb");
    TORCH_CHECK(s.gz, "checkpoint: cannot open ", path);
  } else {
    s.fp = fopen(path.c_str(), "wb");
    TORCH_CHECK(s.fp, "checkpoint: cannot open ", path);
  }
  try {
    fdl_write_stream(s, entries, hash32, version);
  } catch (...) {
    if (s.gz) gzclose(s.gz);
    if (s.fp) fclose(s.fp);
    throw;
  }
  if (s.gz) gzclose(s.gz);
  if (s.fp) fclose(s.fp);
}

py::bytes fdl_save_bytes(const std::vector<std::pair<std::string, Tensor>>& entries, const std::string& hash32, uint32_t version) {
  std::string mem;
  ByteSink s;
  s.mem = &mem;
  fdl_write_stream(s, entries, hash32, version);
  return py::bytes(mem);
}

// returns (version, hash bytes, [(name, tensor)])
py::tuple fdl_read_stream(ByteSource& s, bool keys_only) {
  char magic[4];
  s.read(magic, 4);
  TORCH_CHECK(std::memcmp(magic, "FDLC", 4) == 0, "invalid checkpoint: bad magic (expected .fdl checkpoint)");
  const uint32_t version = s.get<uint32_t>();
  TORCH_CHECK(version >= 1 && version <= 2, "unsupported checkpoint version ", version, " (this build supports 1..=2)");
  std::string hash(32, '\0');
  s.read(hash.data(), 32);
  const uint32_t count = s.get<uint32_t>();
  py::list out;
  for (uint32_t i = 0; i < count; ++i) {
    const uint32_t nl = s.get<uint32_t>();
    TORCH_CHECK(nl < (1u << 20), "checkpoint: implausible name length");
    std::string name(nl, '\0');
    s.read(name.data(), nl);
    Tensor t = read_tensor_record(s, keys_only);
    if (keys_only) out.append(py::make_tuple(name, py::none()));
    else out.append(py::make_tuple(name, t));
  }
  return py::make_tuple(version, py::bytes(hash), out);
}

py::tuple fdl_load(const std::string& path, bool keys_only) {
  ByteSource s;
  s.gz = gzopen(path.c_str(), "rb");  // gzopen reads plain files transparently
  TORCH_CHECK(s.gz, "checkpoint: cannot open ", path);
  try {
    py::tuple r = fdl_read_stream(s, keys_only);
    gzclose(s.gz);
    return r;
  } catch (...) {
    gzclose(s.gz);
    throw;
  }
}
py::tuple fdl_load_bytes(const std::string& data, bool keys_only) {
  ByteSource s;
  s.mem = &data;
  return fdl_read_stream(s, keys_only);
}

// Optimizer-state streams reuse the tensor record with a presence byte.
py::bytes pack_tensor_record(const std::optional<Tensor>& t) {
  std::string mem;
  ByteSink s;
  s.mem = &mem;
  if (!t.has_value() || !t->defined()) {
    s.put<uint8_t>(0);
  } else {
    s.put<uint8_t>(1);
    write_tensor_record(s, *t);
  }
  return py::bytes(mem);
}
py::tuple unpack_tensor_record(const std::string& data, size_t pos) {
  ByteSource s;
  s.mem = &data;
  s.pos = pos;
  const uint8_t present = s.get<uint8_t>();
  if (!present) return py::make_tuple(py::none(), s.pos);
  Tensor t = read_tensor_record(s);
  return py::make_tuple(t, s.pos);
}

// =========================================================================== Xoshiro256++ RNG
// Same generator family as the reference's CPU RNG (flodl/src/rng.rs wraps Xoshiro256++), seeded
// with SplitMix64. Used for epoch shuffles so every rank derives the same permutation from
// (seed, epoch) without communication.
struct Rng {
  uint64_t s[4];
  bool has_spare = false;
  double spare = 0.0;
  explicit Rng(uint64_t seed) {
    uint64_t z = seed;
    for (auto& x : s) {
      z += 0x9E3779B97F4A7C15ull;
      uint64_t r = z;
      r = (r ^ (r >> 30)) * 0xBF58476D1CE4E5B9ull;
      r = (r ^ (r >> 27)) * 0x94D049BB133111EBull;
      x = r ^ (r >> 31);
    }
  }
  static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
  uint64_t next() {
    const uint64_t result = rotl(s[0] + s[3], 23) + s[0];
    const uint64_t t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3];
    s[2] ^= t;
    s[3] = rotl(s[3], 45);
    return result;
  }
  // unbiased integer in [0, n) (Lemire's multiply-shift with rejection)
  uint64_t below(uint64_t n) {
    TORCH_CHECK(n > 0, "Rng.usize(0) is undefined");
    uint64_t x = next();
    __uint128_t m = static_cast<__uint128_t>(x) * n;
    uint64_t l = static_cast<uint64_t>(m);
    if (l < n) {
      const uint64_t t = (0 - n) % n;
      while (l < t) {
        x = next();
        m = static_cast<__uint128_t>(x) * n;
        l = static_cast<uint64_t>(m);
      }
    }
    return static_cast<uint64_t>(m >> 64);
  }
  double f64() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
  float f32() { return (next() >> 40) * (1.0f / 16777216.0f); }
  bool bernoulli(double p) { return f64() < p; }
  int64_t range(int64_t lo, int64_t hi) {
    TORCH_CHECK(hi > lo, "Rng.range: empty range");
    return lo + static_cast<int64_t>(below(static_cast<uint64_t>(hi - lo)));
  }
  double normal(double mean, double stdv) {
    if (has_spare) { has_spare = false; return mean + stdv * spare; }
    double u, v, q;
    do {
      u = 2.0 * f64() - 1.0;
      v = 2.0 * f64() - 1.0;
      q = u * u + v * v;
    } while (q >= 1.0 || q == 0.0);
    const double f = std::sqrt(-2.0 * std::log(q) / q);
    spare = v * f;
    has_spare = true;
    return mean + stdv * u * f;
  }
  // Fisher-Yates over 0..n-1
  Tensor permutation(int64_t n) {
    Tensor t = torch::arange(n, torch::kLong);
    int64_t* p = t.data_ptr<int64_t>();
    for (int64_t i = n - 1; i > 0; --i) std::swap(p[i], p[below(static_cast<uint64_t>(i + 1))]);
    return t;
  }
  std::vector<int64_t> shuffle(std::vector<int64_t> v) {
    for (int64_t i = static_cast<int64_t>(v.size()) - 1; i > 0; --i) std::swap(v[i], v[below(static_cast<uint64_t>(i + 1))]);
    return v;
  }
};

// ============================================================================ prefetch worker
// A background thread assembles batches (row gather into pinned staging) and ships them to the
// device on its own copy stream; a CUDA event per batch lets the consumer's stream wait without
// blocking the host. Counterpart of flodl/src/data/prefetch.rs:163-285.
struct PrefetchWorker {
  std::vector<Tensor> sources;  // CPU tensors, same dim-0 length
  int device;                   // -1 = keep on CPU
  size_t depth;
  std::thread th;
  std::mutex mu;
  std::condition_variable cv_put, cv_get;
  struct Item {
    std::vector<Tensor> tensors;
    std::shared_ptr<at::cuda::CUDAEvent> ready;
  };
  std::deque<Item> queue;
  bool epoch_done = true, stop_flag = false;
  std::string error;
  std::optional<c10::cuda::CUDAStream> copy_stream;

  PrefetchWorker(std::vector<Tensor> src, int dev, size_t depth_) : sources(std::move(src)), device(dev), depth(std::max<size_t>(1, depth_)) {
    TORCH_CHECK(!sources.empty(), "PrefetchWorker needs at least one source tensor");
    for (auto& t : sources) TORCH_CHECK(!t.is_cuda() && t.size(0) == sources[0].size(0), "sources must be CPU tensors with equal length");
    if (device >= 0) copy_stream = c10::cuda::getStreamFromPool(/*isHighPriority=*/false, static_cast<c10::DeviceIndex>(device));
  }
  ~PrefetchWorker() { stop(); }

  void stop() {
    {
      std::lock_guard<std::mutex> g(mu);
      stop_flag = true;
    }
    cv_put.notify_all();
    cv_get.notify_all();
    if (th.joinable()) {
      py::gil_scoped_release rel;
      th.join();
    }
  }

  void start_epoch(const Tensor& order, int64_t batch_size, bool drop_last) {
    TORCH_CHECK(order.scalar_type() == at::kLong && !order.is_cuda() && order.dim() == 1);
    TORCH_CHECK(batch_size > 0);
    stop();
    {
      std::lock_guard<std::mutex> g(mu);
      stop_flag = false;
      epoch_done = false;
      queue.clear();
      error.clear();
    }
    Tensor ord = order.contiguous();
    th = std::thread([this, ord, batch_size, drop_last] { run(ord, batch_size, drop_last); });
  }

  void run(Tensor order, int64_t bs, bool drop_last) {
    try {
      const int64_t n = order.numel();
      for (int64_t off = 0; off < n; off += bs) {
        const int64_t len = std::min(bs, n - off);
        if (len < bs && drop_last) break;
        Tensor idx = order.narrow(0, off, len);
        Item item;
        if (device >= 0) {
          c10::cuda::CUDAGuard dg(static_cast<c10::DeviceIndex>(device));
          c10::cuda::CUDAStreamGuard sg(*copy_stream);
          for (auto& src : sources) {
            std::vector<int64_t> shape = src.sizes().vec();
            shape[0] = len;
            Tensor staged = torch::empty(shape, src.options().pinned_memory(true));
            at::index_select_out(staged, src, 0, idx);
            item.tensors.push_back(staged.to(torch::Device(torch::kCUDA, device), /*non_blocking=*/true));
          }
          item.ready = std::make_shared<at::cuda::CUDAEvent>();
          item.ready->record(*copy_stream);
        } else {
          for (auto& src : sources) item.tensors.push_back(src.index_select(0, idx));
        }
        std::unique_lock<std::mutex> lk(mu);
        cv_put.wait(lk, [this] { return stop_flag || queue.size() < depth; });
        if (stop_flag) return;
        queue.push_back(std::move(item));
        cv_get.notify_one();
      }
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> g(mu);
      error = e.what();
    }
    std::lock_guard<std::mutex> g(mu);
    epoch_done = true;
    cv_get.notify_all();
  }

  // Next batch, or None at the end of the epoch. The current stream is made to wait for the copy.
  py::object next() {
    Item item;
    {
      py::gil_scoped_release rel;
      std::unique_lock<std::mutex> lk(mu);
      cv_get.wait(lk, [this] { return stop_flag || !queue.empty() || epoch_done; });
      if (queue.empty()) {
        lk.unlock();
        py::gil_scoped_acquire acq;
        TORCH_CHECK(error.empty(), "prefetch worker failed: ", error);
        return py::none();
      }
      item = std::move(queue.front());
      queue.pop_front();
      cv_put.notify_one();
    }
    if (item.ready) {
      auto cur = c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device));
      item.ready->block(cur);
      for (auto& t : item.tensors) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cur);
    }
    py::list out;
    for (auto& t : item.tensors) out.append(t);
    return std::move(out);
  }
};

// ==================================================================================== El Che
// Heterogeneous-cadence scheduler (behaviour of flodl/src/distributed/el_che.rs:35-384): the
// slowest device runs `anchor` batches between synchronisations, faster devices proportionally
// more; timings are smoothed with an error-scaled EMA, the anchor grows when synchronisation
// overhead exceeds the target and decays by one when it is under half of it.
struct ElChe {
  size_t world;
  size_t anchor_, min_anchor, max_anchor = 200;
  std::vector<size_t> counts;
  std::vector<double> ms;
  bool calibrated = false;
  double overhead_target = 0.10;
  std::optional<size_t> max_diff;

  ElChe(size_t world_size, size_t anchor) : world(world_size), anchor_(anchor), min_anchor(anchor), counts(world_size, anchor), ms(world_size, 0.0) {
    TORCH_CHECK(world_size >= 2, "El Che requires at least 2 devices");
    TORCH_CHECK(anchor >= 1, "anchor must be >= 1");
  }
  void set_overhead_target(double t) { overhead_target = std::clamp(t, 0.01, 0.50); }
  void set_max_anchor(size_t m) {
    max_anchor = std::max<size_t>(m, 1);
    if (min_anchor > max_anchor) {
      min_anchor = max_anchor;
      anchor_ = std::clamp(anchor_, min_anchor, max_anchor);
    }
  }
  void set_max_batch_diff(size_t m) { max_diff = m; }
  void set_speed_ratio(size_t slow_rank, double ratio) {
    TORCH_CHECK(slow_rank < world, "slow_rank (", slow_rank, ") out of bounds for world_size (", world, ")");
    ratio = std::max(ratio, 1.0);
    for (size_t r = 0; r < world; ++r)
      counts[r] = (r == slow_rank) ? anchor_ : static_cast<size_t>(std::max(1.0, std::round(anchor_ * ratio)));
  }
  double slowest() const { return ms.empty() ? 0.0 : *std::max_element(ms.begin(), ms.end()); }
  double anchor_wall_ms() const { return calibrated ? anchor_ * slowest() : 0.0; }
  size_t total() const { size_t s = 0; for (auto c : counts) s += c; return s; }
  bool has_speed_hint() const {
    for (size_t i = 1; i < counts.size(); ++i) if (counts[i] != counts[i - 1]) return true;
    return false;
  }
  void recompute(double slow_ms) {
    for (size_t r = 0; r < world; ++r) {
      size_t target = anchor_;
      if (ms[r] > 0.0 && std::fabs(ms[r] - slow_ms) >= 1e-6)
        target = static_cast<size_t>(std::max(1.0, std::round(anchor_ * (slow_ms / ms[r]))));
      const size_t cur = counts[r];
      const double diff = std::fabs(double(target) - double(cur));
      if (diff > cur * 0.10 || !calibrated) {
        size_t next = target;
        if (max_diff.has_value() && calibrated) {
          if (target > cur) next = std::min(cur + *max_diff, target);
          else next = std::max<size_t>(std::max(cur > *max_diff ? cur - *max_diff : 0, target), 1);
        }
        counts[r] = next;
      }
    }
  }
  void nudge_anchor_down(double factor) {
    const size_t nw = static_cast<size_t>(std::ceil(anchor_ * std::clamp(factor, 0.1, 1.0)));
    anchor_ = std::min(std::max<size_t>(nw, 1), anchor_);
    const double s = slowest();
    if (s > 0.0) recompute(s);
  }
  void report_timing(const std::vector<double>& wall_ms, const std::vector<size_t>& batches, double sync_ms) {
    TORCH_CHECK(wall_ms.size() == world, "wall_ms length must match world_size");
    for (size_t r = 0; r < world; ++r) {
      const size_t n = r < batches.size() ? batches[r] : 0;
      if (n > 0 && wall_ms[r] > 0.0) {
        const double fresh = wall_ms[r] / n;
        if (calibrated && ms[r] > 0.0) {
          const double a = std::clamp(std::fabs(fresh - ms[r]) / ms[r], 0.1, 0.8);
          ms[r] = a * fresh + (1.0 - a) * ms[r];
        } else {
          ms[r] = fresh;
        }
      }
    }
    const double slow_ms = slowest();
    if (slow_ms <= 0.0) return;
    const double compute_ms = *std::max_element(wall_ms.begin(), wall_ms.end());
    if (compute_ms > 0.0 && sync_ms > 0.0) {
      const double overhead = sync_ms / compute_ms;
      if (overhead > overhead_target) {
        const size_t grown = static_cast<size_t>(std::ceil(anchor_ * (overhead / overhead_target)));
        anchor_ = std::clamp(grown, min_anchor, max_anchor);
      } else if (overhead < overhead_target * 0.5 && anchor_ > min_anchor) {
        anchor_ -= 1;
      }
    }
    recompute(slow_ms);
    calibrated = true;
  }
  std::vector<size_t> clamp_total(size_t max_total) const {
    const size_t cur = total();
    if (cur <= max_total) return counts;
    const double scale = double(max_total) / double(cur);
    std::vector<size_t> out(world);
    size_t sum = 0;
    for (size_t r = 0; r < world; ++r) {
      out[r] = static_cast<size_t>(std::max(1.0, std::floor(counts[r] * scale)));
      sum += out[r];
    }
    size_t rem = max_total > sum ? max_total - sum : 0;
    for (auto& c : out) {
      if (!rem) break;
      c += 1;
      rem -= 1;
    }
    return out;
  }
};

}  // namespace

// Kahn levels of a DAG given as (from, to) node-index pairs (flodl/src/graph/graph.rs:180-260): level k holds
// the nodes whose last dependency sits in level k-1; inside a level nodes appear in the order their last
// dependency released them (dependents visited in ascending index). Duplicate edges count once. Throws on a cycle.
static std::vector<std::vector<int64_t>> topo_levels(int64_t n, const std::vector<std::pair<int64_t, int64_t>>& edges) {
  if (n < 0) throw std::runtime_error("topo_levels: negative node count");
  std::vector<std::set<int64_t>> deps(n), dependents(n);
  for (const auto& e : edges) {
    if (e.first < 0 || e.first >= n || e.second < 0 || e.second >= n) throw std::runtime_error("topo_levels: edge endpoint out of range");
    deps[e.second].insert(e.first);
    dependents[e.first].insert(e.second);
  }
  std::vector<int64_t> indeg(n), queue;
  for (int64_t i = 0; i < n; ++i) {
    indeg[i] = static_cast<int64_t>(deps[i].size());
    if (indeg[i] == 0) queue.push_back(i);
  }
  std::vector<std::vector<int64_t>> levels;
  int64_t visited = 0;
  while (!queue.empty()) {
    levels.push_back(queue);
    visited += static_cast<int64_t>(queue.size());
    std::vector<int64_t> next;
    for (int64_t ni : queue)
      for (int64_t d : dependents[ni])
        if (--indeg[d] == 0) next.push_back(d);
    queue.swap(next);
  }
  if (visited != n) throw std::runtime_error("cycle detected in graph");
  return levels;
}

void bind_runtime(py::module_& m) {
  m.def("topo_levels", &topo_levels, py::arg("n"), py::arg("edges"));
  m.def("sha256_hex", [](py::bytes b) { return sha256_hex(std::string(b)); });
  m.def("fdl_save", &fdl_save, py::arg("path"), py::arg("entries"), py::arg("hash32"), py::arg("version") = 2);
  m.def("fdl_save_bytes", &fdl_save_bytes, py::arg("entries"), py::arg("hash32"), py::arg("version") = 2);
  m.def("fdl_load", &fdl_load, py::arg("path"), py::arg("keys_only") = false);
  m.def("fdl_load_bytes", [](py::bytes b, bool keys_only) { return fdl_load_bytes(std::string(b), keys_only); }, py::arg("data"),
        py::arg("keys_only") = false);
  m.def("pack_tensor_record", &pack_tensor_record);
  m.def("unpack_tensor_record", [](py::bytes b, size_t pos) { return unpack_tensor_record(std::string(b), pos); });

  py::class_<Rng>(m, "Rng")
      .def(py::init<uint64_t>())
      .def_static("seed", [](uint64_t s) { return Rng(s); })
      .def("usize", &Rng::below)
      .def("next_u64", &Rng::next)
      .def("f32", &Rng::f32)
      .def("f64", &Rng::f64)
      .def("bernoulli", &Rng::bernoulli)
      .def("range", &Rng::range)
      .def("normal", &Rng::normal)
      .def("permutation", &Rng::permutation)
      .def("shuffle", &Rng::shuffle)
      .def("clone", [](const Rng& r) { return Rng(r); });

  py::class_<PrefetchWorker>(m, "PrefetchWorker")
      .def(py::init<std::vector<Tensor>, int, size_t>(), py::arg("sources"), py::arg("device"), py::arg("depth") = 4)
      .def("start_epoch", &PrefetchWorker::start_epoch, py::arg("order"), py::arg("batch_size"), py::arg("drop_last") = true)
      .def("next", &PrefetchWorker::next)
      .def("stop", &PrefetchWorker::stop);

  py::class_<ElChe>(m, "ElChe")
      .def(py::init<size_t, size_t>(), py::arg("world_size"), py::arg("anchor"))
      .def("set_overhead_target", &ElChe::set_overhead_target)
      .def("set_max_anchor", &ElChe::set_max_anchor)
      .def("set_max_batch_diff", &ElChe::set_max_batch_diff)
      .def("set_speed_ratio", &ElChe::set_speed_ratio)
      .def("batches", [](const ElChe& e, size_t r) { return e.counts.at(r); })
      .def("batch_counts", [](const ElChe& e) { return e.counts; })
      .def("total_batches", &ElChe::total)
      .def("anchor", [](const ElChe& e) { return e.anchor_; })
      .def("anchor_wall_ms", &ElChe::anchor_wall_ms)
      .def("nudge_anchor_down", &ElChe::nudge_anchor_down)
      .def("is_calibrated", [](const ElChe& e) { return e.calibrated; })
      .def("has_speed_hint", &ElChe::has_speed_hint)
      .def("ms_per_batch", [](const ElChe& e) { return e.ms; })
      .def("max_batch_diff", [](const ElChe& e) -> py::object { return e.max_diff ? py::cast(*e.max_diff) : py::none(); })
      .def("report_timing", &ElChe::report_timing, py::arg("wall_ms"), py::arg("actual_batches"), py::arg("sync_ms"))
      .def("clamp_total", &ElChe::clamp_total);
}
