// Host-side SwiGLU expert FFN for GPU misses of the expert tiers, plus the persistent worker pool
// that runs one job per (expert, rows) and a direct-IO reader pool for the NVMe tier.
//
//   y[r] = bf16( silu_mul( bf16(x[r] · Wgu^T) ) · Wd^T )        (BF16 storage, FP32 accumulation)
//
// Three arms selected at run time (cpuid): AVX-512F, AVX2+FMA, scalar; they accumulate in the same
// order class (8 / 16 lane partial sums, then a fixed horizontal tree), and the test-suite checks
// them against each other and against the PyTorch oracle. The reference implements the same role
// in src/cpu/expert_ffn.rs (scalar / AVX2+FMA / AVX-512-BF16 arms, persistent pool with pre-wake
// spin, service-time table for the planner) and src/experts/disk.rs (O_DIRECT aligned reads into a
// pinned ring, one reader thread per slot).
#include <immintrin.h>
#include <stdint.h>
#include <string.h>
#include <math.h>
#include <fcntl.h>
#include <unistd.h>
#include <errno.h>
#include <stdlib.h>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#define FF_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bf16_to_f32(uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint16_t f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);     // NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                              // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float bf16_round(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// ---- dot products of a BF16 weight row with an FP32 activation row ---------------------------
float dot_scalar(const uint16_t* w, const float* x, int n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] = fmaf(bf16_to_f32(w[i + j]), x[i + j], acc[j]);
  float tail = 0.f;
  for (; i < n; ++i) tail = fmaf(bf16_to_f32(w[i]), x[i], tail);
  return (((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]))) + tail;
}

__attribute__((target("avx2,fma")))
float dot_avx2(const uint16_t* w, const float* x, int n) {
  __m256 acc = _mm256_setzero_ps();
  int i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m128i wb = _mm_loadu_si128((const __m128i*)(w + i));
    const __m256 wf = _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(wb), 16));
    acc = _mm256_fmadd_ps(wf, _mm256_loadu_ps(x + i), acc);
  }
  float a[8]; _mm256_storeu_ps(a, acc);
  float tail = 0.f;
  for (; i < n; ++i) tail = fmaf(bf16_to_f32(w[i]), x[i], tail);
  return (((a[0] + a[4]) + (a[2] + a[6])) + ((a[1] + a[5]) + (a[3] + a[7]))) + tail;
}

__attribute__((target("avx512f,avx512bw")))
float dot_avx512(const uint16_t* w, const float* x, int n) {
  __m512 acc = _mm512_setzero_ps();
  int i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m256i wb = _mm256_loadu_si256((const __m256i*)(w + i));
    const __m512 wf = _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(wb), 16));
    acc = _mm512_fmadd_ps(wf, _mm512_loadu_ps(x + i), acc);
  }
  float tail = 0.f;
  for (; i < n; ++i) tail = fmaf(bf16_to_f32(w[i]), x[i], tail);
  return _mm512_reduce_add_ps(acc) + tail;
}

typedef float (*DotFn)(const uint16_t*, const float*, int);

int detect_arm() {
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) return 2;
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 1;
  return 0;
}
DotFn dot_for(int arm) { return arm == 2 ? dot_avx512 : arm == 1 ? dot_avx2 : dot_scalar; }

inline float silu(float v) { return v / (1.0f + expf(-v)); }

// one expert over `rows` token rows. wgu: [2f, h] rows [gate | up]; wd: [h, f]
void expert_ffn(const uint16_t* x, int ldx, const uint16_t* wgu, const uint16_t* wd, uint16_t* y, int ldy, int rows,
                int h, int f, int mode, int arm) {
  const DotFn dot = dot_for(arm);
  std::vector<float> xf(h), mid(f);
  for (int r = 0; r < rows; ++r) {
    for (int i = 0; i < h; ++i) xf[i] = bf16_to_f32(x[(size_t)r * ldx + i]);
    for (int j = 0; j < f; ++j) {
      const float g = bf16_round(dot(wgu + (size_t)j * h, xf.data(), h));
      const float u = bf16_round(dot(wgu + (size_t)(f + j) * h, xf.data(), h));
      const float a = mode == 0 ? bf16_round(silu(g)) * u : silu(g) * u;
      mid[j] = bf16_round(a);
    }
    for (int i = 0; i < h; ++i) y[(size_t)r * ldy + i] = f32_to_bf16(dot(wd + (size_t)i * f, mid.data(), f));
  }
}

// ---- worker pool -------------------------------------------------------------------------------
struct Job {
  const uint16_t* x; int ldx; const uint16_t* wgu; const uint16_t* wd; uint16_t* y; int ldy; int rows, h, f, mode;
};

struct Pool {
  std::vector<std::thread> threads;
  std::mutex mu;
  std::condition_variable cv, done_cv;
  const Job* jobs = nullptr;
  int n_jobs = 0;
  std::atomic<int> next{0};
  int finished = 0, generation = 0;
  bool stop = false;
  int arm = 0;

  explicit Pool(int n, int arm_) : arm(arm_) {
    for (int i = 0; i < n; ++i) threads.emplace_back([this] { loop(); });
  }
  ~Pool() {
    { std::lock_guard<std::mutex> l(mu); stop = true; }
    cv.notify_all();
    for (auto& t : threads) t.join();
  }
  void loop() {
    int seen = 0;
    while (true) {
      {
        std::unique_lock<std::mutex> l(mu);
        cv.wait(l, [&] { return stop || generation != seen; });
        if (stop) return;
        seen = generation;
      }
      work();
      {
        std::lock_guard<std::mutex> l(mu);
        if (++finished == (int)threads.size()) done_cv.notify_all();
      }
    }
  }
  void work() {
    while (true) {
      const int i = next.fetch_add(1);
      if (i >= n_jobs) return;
      const Job& j = jobs[i];
      expert_ffn(j.x, j.ldx, j.wgu, j.wd, j.y, j.ldy, j.rows, j.h, j.f, j.mode, arm);
    }
  }
  void run(const Job* js, int n) {
    {
      std::lock_guard<std::mutex> l(mu);
      jobs = js; n_jobs = n; next = 0; finished = 0; ++generation;
    }
    cv.notify_all();
    std::unique_lock<std::mutex> l(mu);
    done_cv.wait(l, [&] { return finished == (int)threads.size(); });
  }
};

// ---- direct-IO reader pool ---------------------------------------------------------------------
struct ReadReq { int fd; long long offset; long long len; void* dst; int ticket; };

struct Reader {
  std::vector<std::thread> threads;
  std::mutex mu;
  std::condition_variable cv, done_cv;
  std::deque<ReadReq> q;
  std::vector<int> status;            // per ticket: 0 pending, 1 ok, <0 -errno
  bool stop = false;
  std::atomic<int> in_flight{0};
  static constexpr long long ALIGN = 4096;

  explicit Reader(int n) { for (int i = 0; i < n; ++i) threads.emplace_back([this] { loop(); }); }
  ~Reader() {
    { std::lock_guard<std::mutex> l(mu); stop = true; }
    cv.notify_all();
    for (auto& t : threads) t.join();
  }
  static int do_read(const ReadReq& r) {
    // O_DIRECT needs aligned offset, length and buffer: read the aligned superset into a bounce
    // buffer when the request is not aligned, straight into dst when it is
    const long long a0 = r.offset / ALIGN * ALIGN;
    const long long a1 = (r.offset + r.len + ALIGN - 1) / ALIGN * ALIGN;
    const bool direct_ok = (r.offset % ALIGN == 0) && (r.len % ALIGN == 0) && (((uintptr_t)r.dst) % ALIGN == 0);
    void* buf = r.dst;
    if (!direct_ok) { if (posix_memalign(&buf, ALIGN, (size_t)(a1 - a0))) return -ENOMEM; }
    long long got = 0;
    const long long want = direct_ok ? r.len : a1 - a0;
    const long long base = direct_ok ? r.offset : a0;
    while (got < want) {
      const ssize_t n = pread(r.fd, (char*)buf + got, (size_t)(want - got), base + got);
      if (n < 0) { if (errno == EINTR) continue; const int e = errno; if (!direct_ok) free(buf); return -e; }
      if (n == 0) break;                                  // end of file inside the aligned tail
      got += n;
    }
    if (!direct_ok) {
      if (got < (r.offset - a0) + r.len) { free(buf); return -EIO; }
      memcpy(r.dst, (char*)buf + (r.offset - a0), (size_t)r.len);
      free(buf);
    } else if (got < r.len) return -EIO;
    return 1;
  }
  void loop() {
    while (true) {
      ReadReq r;
      {
        std::unique_lock<std::mutex> l(mu);
        cv.wait(l, [&] { return stop || !q.empty(); });
        if (stop && q.empty()) return;
        r = q.front(); q.pop_front();
      }
      const int st = do_read(r);
      {
        std::lock_guard<std::mutex> l(mu);
        status[r.ticket] = st;
        in_flight--;
      }
      done_cv.notify_all();
    }
  }
  int submit(int fd, long long off, long long len, void* dst) {
    std::lock_guard<std::mutex> l(mu);
    const int t = (int)status.size();
    status.push_back(0);
    q.push_back({fd, off, len, dst, t});
    in_flight++;
    cv.notify_one();
    return t;
  }
  int wait(int ticket, int timeout_ms) {
    std::unique_lock<std::mutex> l(mu);
    if (ticket < 0 || ticket >= (int)status.size()) return -EINVAL;
    if (!done_cv.wait_for(l, std::chrono::milliseconds(timeout_ms), [&] { return status[ticket] != 0; })) return 0;
    return status[ticket];
  }
};

}  // namespace

FF_API int ff_cpu_arm() { static int arm = detect_arm(); return arm; }

// arm: -1 = best available, 0 scalar, 1 AVX2+FMA, 2 AVX-512
FF_API int ff_cpu_expert_ffn(const uint16_t* x, int ldx, const uint16_t* wgu, const uint16_t* wd, uint16_t* y, int ldy,
                             int rows, int h, int f, int mode, int arm) {
  if (rows < 0 || h <= 0 || f <= 0) return -1;
  const int best = ff_cpu_arm();
  if (arm < 0 || arm > best) arm = arm < 0 ? best : -2;
  if (arm == -2) return -2;                                 // requested arm not supported by this CPU
  expert_ffn(x, ldx, wgu, wd, y, ldy, rows, h, f, mode, arm);
  return 0;
}

FF_API void* ff_pool_create(int threads) {
  if (threads < 1) threads = 1;
  return new Pool(threads, ff_cpu_arm());
}
FF_API void ff_pool_destroy(void* p) { delete static_cast<Pool*>(p); }

// jobs: array of n records {x, ldx, wgu, wd, y, ldy, rows, h, f, mode} laid out as below
struct FfJob { const uint16_t* x; long long ldx; const uint16_t* wgu; const uint16_t* wd; uint16_t* y; long long ldy;
               int rows, h, f, mode; };
FF_API int ff_pool_run(void* p, const FfJob* jobs, int n) {
  if (!p || n < 0) return -1;
  std::vector<Job> js(n);
  for (int i = 0; i < n; ++i)
    js[i] = Job{jobs[i].x, (int)jobs[i].ldx, jobs[i].wgu, jobs[i].wd, jobs[i].y, (int)jobs[i].ldy, jobs[i].rows,
                jobs[i].h, jobs[i].f, jobs[i].mode};
  static_cast<Pool*>(p)->run(js.data(), n);
  return 0;
}

// ---- direct IO ---------------------------------------------------------------------------------
FF_API int ff_dio_open(const char* path, int direct) {
  int fd = -1;
  if (direct) fd = open(path, O_RDONLY | O_DIRECT | O_CLOEXEC);
  if (fd < 0) fd = open(path, O_RDONLY | O_CLOEXEC);        // filesystems without O_DIRECT (tmpfs)
  return fd < 0 ? -errno : fd;
}
FF_API void ff_dio_close(int fd) { if (fd >= 0) close(fd); }
FF_API void* ff_reader_create(int threads) { return new Reader(threads < 1 ? 1 : threads); }
FF_API void ff_reader_destroy(void* r) { delete static_cast<Reader*>(r); }
FF_API int ff_reader_submit(void* r, int fd, long long offset, long long len, void* dst) {
  if (!r || fd < 0 || offset < 0 || len <= 0 || !dst) return -EINVAL;
  return static_cast<Reader*>(r)->submit(fd, offset, len, dst);
}
// returns 1 done, 0 still pending after timeout_ms, < 0 -errno
FF_API int ff_reader_wait(void* r, int ticket, int timeout_ms) { return static_cast<Reader*>(r)->wait(ticket, timeout_ms); }
FF_API int ff_reader_in_flight(void* r) { return static_cast<Reader*>(r)->in_flight.load(); }
