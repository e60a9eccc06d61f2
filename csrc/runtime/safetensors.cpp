// Safetensors byte path: mmap reader with multi-threaded F32/F16/BF16 -> fp32 decode, and an
// incremental writer (header first, then tensor payloads appended in order, fsync + atomic rename).
// The JSON header itself is produced/parsed by the Python layer; this file moves the bytes.
// Reference: crates/checkpoint/src/st.rs:216-308 (dtype decode, tmp+rename),
// crates/checkpoint/src/weightio.rs:48-235 (streaming reader), :387-551 (incremental writer).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#define BBH_API extern "C" __attribute__((visibility("default")))

namespace {

struct Mapped {
  int fd = -1;
  uint8_t* base = nullptr;
  size_t size = 0;
  uint64_t header_len = 0;
};

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      u = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_f16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

template <typename F>
void parallel_for(int64_t n, F fn) {
  const int64_t min_chunk = 1 << 18;
  int nt = static_cast<int>(std::min<int64_t>(std::thread::hardware_concurrency(), (n + min_chunk - 1) / min_chunk));
  if (nt <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> ts;
  const int64_t per = (n + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int64_t a = t * per, b = std::min<int64_t>(n, a + per);
    if (a >= b) break;
    ts.emplace_back([=] { fn(a, b); });
  }
  for (auto& t : ts) t.join();
}

struct Writer {
  FILE* f = nullptr;
  std::string tmp;
  uint64_t written = 0;
};

}  // namespace

// ---- reader -------------------------------------------------------------------------------
BBH_API void* bbh_st_map(const char* path) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (p == MAP_FAILED) {
    ::close(fd);
    return nullptr;
  }
  auto* m = new Mapped();
  m->fd = fd;
  m->base = static_cast<uint8_t*>(p);
  m->size = st.st_size;
  std::memcpy(&m->header_len, m->base, 8);  // little-endian u64
  if (m->header_len > m->size - 8) {
    munmap(p, st.st_size);
    ::close(fd);
    delete m;
    return nullptr;
  }
  return m;
}
BBH_API void bbh_st_unmap(void* h) {
  auto* m = static_cast<Mapped*>(h);
  if (!m) return;
  munmap(m->base, m->size);
  ::close(m->fd);
  delete m;
}
BBH_API uint64_t bbh_st_header_len(void* h) { return static_cast<Mapped*>(h)->header_len; }
BBH_API const char* bbh_st_header_ptr(void* h) {
  return reinterpret_cast<const char*>(static_cast<Mapped*>(h)->base + 8);
}
BBH_API uint64_t bbh_st_data_bytes(void* h) {
  auto* m = static_cast<Mapped*>(h);
  return m->size - 8 - m->header_len;
}
// Decode `n` elements at data offset `begin` (relative to the data section) to fp32.
// dtype: 0 F32, 1 F16, 2 BF16.  Returns 0, -1 out of range, -2 unknown dtype.
BBH_API int bbh_st_decode_f32(void* h, uint64_t begin, int64_t n, int dtype, float* dst) {
  auto* m = static_cast<Mapped*>(h);
  const int es = dtype == 0 ? 4 : 2;
  if (dtype < 0 || dtype > 2) return -2;
  const uint64_t data0 = 8 + m->header_len;
  if (data0 + begin + static_cast<uint64_t>(n) * es > m->size) return -1;
  const uint8_t* src = m->base + data0 + begin;
  if (dtype == 0) {
    parallel_for(n, [=](int64_t a, int64_t b) { std::memcpy(dst + a, src + a * 4, (b - a) * 4); });
  } else if (dtype == 1) {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    parallel_for(n, [=](int64_t a, int64_t b) {
      for (int64_t i = a; i < b; ++i) dst[i] = f16_to_f32(s[i]);
    });
  } else {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    parallel_for(n, [=](int64_t a, int64_t b) {
      for (int64_t i = a; i < b; ++i) dst[i] = bf16_to_f32(s[i]);
    });
  }
  return 0;
}
BBH_API int bbh_st_read_raw(void* h, uint64_t begin, uint64_t nbytes, void* dst) {
  auto* m = static_cast<Mapped*>(h);
  const uint64_t data0 = 8 + m->header_len;
  if (data0 + begin + nbytes > m->size) return -1;
  std::memcpy(dst, m->base + data0 + begin, nbytes);
  return 0;
}

// ---- writer -------------------------------------------------------------------------------
BBH_API void* bbh_stw_open(const char* final_path, const char* header, uint64_t header_len) {
  auto* w = new Writer();
  w->tmp = std::string(final_path) + ".tmp";
  w->f = std::fopen(w->tmp.c_str(), "wb");
  if (!w->f) {
    delete w;
    return nullptr;
  }
  std::fwrite(&header_len, 8, 1, w->f);
  std::fwrite(header, 1, header_len, w->f);
  return w;
}
// Append n fp32 values encoded as dtype (0 F32, 1 F16, 2 BF16).
BBH_API int bbh_stw_append_f32(void* h, const float* src, int64_t n, int dtype) {
  auto* w = static_cast<Writer*>(h);
  if (dtype == 0) {
    if (std::fwrite(src, 4, n, w->f) != static_cast<size_t>(n)) return -1;
    w->written += n * 4;
    return 0;
  }
  std::vector<uint16_t> buf(static_cast<size_t>(n));
  uint16_t* d = buf.data();
  if (dtype == 1)
    parallel_for(n, [=](int64_t a, int64_t b) { for (int64_t i = a; i < b; ++i) d[i] = f32_to_f16(src[i]); });
  else if (dtype == 2)
    parallel_for(n, [=](int64_t a, int64_t b) { for (int64_t i = a; i < b; ++i) d[i] = f32_to_bf16(src[i]); });
  else
    return -2;
  if (std::fwrite(d, 2, n, w->f) != static_cast<size_t>(n)) return -1;
  w->written += n * 2;
  return 0;
}
BBH_API int bbh_stw_append_raw(void* h, const void* src, uint64_t nbytes) {
  auto* w = static_cast<Writer*>(h);
  if (std::fwrite(src, 1, nbytes, w->f) != nbytes) return -1;
  w->written += nbytes;
  return 0;
}
// Flush, fsync and rename <path>.tmp -> <path>.  abort != 0 removes the temporary instead.
BBH_API int bbh_stw_close(void* h, const char* final_path, int abort_write) {
  auto* w = static_cast<Writer*>(h);
  int rc = 0;
  if (std::fflush(w->f) != 0) rc = -1;
  if (fsync(fileno(w->f)) != 0) rc = -1;
  std::fclose(w->f);
  if (abort_write || rc != 0) {
    std::remove(w->tmp.c_str());
  } else if (std::rename(w->tmp.c_str(), final_path) != 0) {
    rc = -2;
  }
  delete w;
  return rc;
}
