// sf_* runtime selection API: per-shape choice between the dense library GEMM and the sparse
// kernels, persisted in an SQLite table.
//
// Behaviour follows the reference runtime (experiments/old_structure/runtime):
//   api/sparseflow_api.cpp:21-63        entry points, NULL path => "kernel_cache.db"
//   dispatch/kernel_dispatcher.cpp:16-28 power-of-two bucketing, min 32, cap 65535
//   dispatch/kernel_dispatcher.cpp:42-188 lookup -> eligibility -> benchmark -> persist
//   dispatch/eligibility_policy.cpp:26-88 four rules: 2:4 only, >= 512^3 flops, quarantine after
//                                         three failures, compressed weight must be cached
//   cache/kernel_cache.cpp:49-99         table schema, WAL journal
//   cache/kernel_key.cpp:7-17            key string "M=..;N=..;K=..;dtype=..;layout=..;sp=..;sm=.."
//   benchmark/micro_bench.cpp:37-49,71-174 L2 flush, 3 warm-up + 10 timed, CV > 5 % => one retry
//
//   cache/compressed_cache.cpp:9-104    content-keyed store of compressed weights (FNV-1a of the first
//                                       KiB of the device matrix + shape), 1 GiB cap; consulted at
//                                       dispatch/kernel_dispatcher.cpp:67-80
//
// Upstream's C entry point passes no matrix (api/sparseflow_api.cpp:44: A = B = C = nullptr), so through
// sf_select_kernel alone its "compression cached" rule can never hold and every 2:4 shape is cached
// as dense; the dispatcher's pointer-taking form is C++ only.  The same is true here for
// sf_select_kernel; sf_select_kernel_ex is the C form of that C++ call (device pointers), and
// sf_compress_weight fills the content-keyed store the way upstream's sparse launcher does
// (kernels/sparse_cusparselt_24.cu:70-89).
//
// Environment: SPARSEFLOW_LOG=1 logs decisions to stderr; SPARSEFLOW_CACHE_DB replaces the default
// database path used for a NULL cache_path; SPARSEFLOW_FORCE=dense|sparse bypasses lookup and
// measurement and returns kernel 0 / 2 for every eligible-by-shape request (nothing is persisted).
//
// Differences, on purpose: the winner is the candidate with the lower measured time (the reference
// halves the sparse flop count before comparing GFLOPS, which makes sparse need a 2x win); each
// store is guarded by its own mutex; libsqlite3 and libcublas are resolved with dlopen at first use
// so the library loads on hosts that lack them (the store then lives in memory only and the dense
// candidate is skipped).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <cmath>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/sparseflow_b200.h"
#include "device_state.h"
#include "kernels.h"

namespace sfb200 {
namespace {

bool log_on() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SPARSEFLOW_LOG");
    v = (e && *e && *e != '0') ? 1 : 0;
  }
  return v == 1;
}
#define SF_LOG(...)                       \
  do {                                    \
    if (log_on()) {                       \
      fprintf(stderr, "[sparseflow] ");   \
      fprintf(stderr, __VA_ARGS__);       \
      fprintf(stderr, "\n");              \
    }                                     \
  } while (0)

// ---------------------------------------------------------------- sqlite via dlopen
struct sqlite3;
struct sqlite3_stmt;
struct SqliteApi {
  int (*open)(const char*, sqlite3**);
  int (*close)(sqlite3*);
  int (*exec)(sqlite3*, const char*, int (*)(void*, int, char**, char**), void*, char**);
  int (*prepare_v2)(sqlite3*, const char*, int, sqlite3_stmt**, const char**);
  int (*bind_text)(sqlite3_stmt*, int, const char*, int, void (*)(void*));
  int (*bind_int)(sqlite3_stmt*, int, int);
  int (*bind_int64)(sqlite3_stmt*, int, long long);
  int (*bind_double)(sqlite3_stmt*, int, double);
  int (*step)(sqlite3_stmt*);
  int (*column_int)(sqlite3_stmt*, int);
  double (*column_double)(sqlite3_stmt*, int);
  int (*finalize)(sqlite3_stmt*);
  void (*free)(void*);
  int (*busy_timeout)(sqlite3*, int);
  bool ok = false;
};
constexpr int kSqliteOk = 0, kSqliteRow = 100, kSqliteDone = 101;
#define SF_SQLITE_TRANSIENT (reinterpret_cast<void (*)(void*)>(-1))

const SqliteApi& sqlite_api() {
  static SqliteApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libsqlite3.so.0", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libsqlite3.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) {
      SF_LOG("libsqlite3 not found: kernel cache is in-memory only");
      return;
    }
    bool all = true;
    auto sym = [&](const char* n) {
      void* p = dlsym(h, n);
      if (!p) all = false;
      return p;
    };
    api.open = reinterpret_cast<decltype(api.open)>(sym("sqlite3_open"));
    api.close = reinterpret_cast<decltype(api.close)>(sym("sqlite3_close"));
    api.exec = reinterpret_cast<decltype(api.exec)>(sym("sqlite3_exec"));
    api.prepare_v2 = reinterpret_cast<decltype(api.prepare_v2)>(sym("sqlite3_prepare_v2"));
    api.bind_text = reinterpret_cast<decltype(api.bind_text)>(sym("sqlite3_bind_text"));
    api.bind_int = reinterpret_cast<decltype(api.bind_int)>(sym("sqlite3_bind_int"));
    api.bind_int64 = reinterpret_cast<decltype(api.bind_int64)>(sym("sqlite3_bind_int64"));
    api.bind_double = reinterpret_cast<decltype(api.bind_double)>(sym("sqlite3_bind_double"));
    api.step = reinterpret_cast<decltype(api.step)>(sym("sqlite3_step"));
    api.column_int = reinterpret_cast<decltype(api.column_int)>(sym("sqlite3_column_int"));
    api.column_double = reinterpret_cast<decltype(api.column_double)>(sym("sqlite3_column_double"));
    api.finalize = reinterpret_cast<decltype(api.finalize)>(sym("sqlite3_finalize"));
    api.free = reinterpret_cast<decltype(api.free)>(sym("sqlite3_free"));
    api.busy_timeout = reinterpret_cast<decltype(api.busy_timeout)>(sym("sqlite3_busy_timeout"));
    api.ok = all;
  });
  return api;
}

struct Entry {
  int kernel = 0;
  double gflops = 0;
  int sparse_failed = 0;
  int failure_count = 0;
};

// Persistent key -> Entry table.  One connection per store; a second connection to the same file
// (sf_cache_size / sf_cache_clear open their own, like the reference) is safe under WAL.
class KernelStore {
 public:
  explicit KernelStore(const std::string& path) : path_(path) {
    const SqliteApi& s = sqlite_api();
    if (!s.ok) return;
    if (s.open(path.c_str(), &db_) != kSqliteOk) {
      SF_LOG("cannot open %s: store is in-memory only", path.c_str());
      if (db_) s.close(db_);
      db_ = nullptr;
      return;
    }
    s.busy_timeout(db_, 2000);
    exec("PRAGMA journal_mode=WAL;");
    exec("PRAGMA synchronous=NORMAL;");
    exec("CREATE TABLE IF NOT EXISTS kernel_cache ("
         " key_hash TEXT PRIMARY KEY,"
         " best_kernel INTEGER NOT NULL,"
         " best_gflops REAL NOT NULL,"
         " sparse_failed INTEGER NOT NULL DEFAULT 0,"
         " failure_count INTEGER NOT NULL DEFAULT 0,"
         " last_failure_code INTEGER NOT NULL DEFAULT 0,"
         " last_failure_ts INTEGER NOT NULL DEFAULT 0);");
    // older files may lack the quarantine columns
    for (const char* col : {"sparse_failed", "failure_count", "last_failure_code", "last_failure_ts"}) {
      if (!has_column(col)) {
        std::string q = std::string("ALTER TABLE kernel_cache ADD COLUMN ") + col +
                        " INTEGER NOT NULL DEFAULT 0;";
        exec(q.c_str());
      }
    }
  }
  ~KernelStore() {
    if (db_) sqlite_api().close(db_);
  }
  KernelStore(const KernelStore&) = delete;
  KernelStore& operator=(const KernelStore&) = delete;

  bool get(const std::string& key, Entry* out) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!db_) {
      auto it = mem_.find(key);
      if (it == mem_.end()) return false;
      *out = it->second;
      return true;
    }
    const SqliteApi& s = sqlite_api();
    sqlite3_stmt* st = nullptr;
    if (s.prepare_v2(db_, "SELECT best_kernel, best_gflops, sparse_failed, failure_count FROM "
                          "kernel_cache WHERE key_hash=?1;", -1, &st, nullptr) != kSqliteOk)
      return false;
    s.bind_text(st, 1, key.c_str(), -1, SF_SQLITE_TRANSIENT);
    bool found = false;
    if (s.step(st) == kSqliteRow) {
      out->kernel = s.column_int(st, 0);
      out->gflops = s.column_double(st, 1);
      out->sparse_failed = s.column_int(st, 2);
      out->failure_count = s.column_int(st, 3);
      found = true;
    }
    s.finalize(st);
    return found;
  }

  bool put_best(const std::string& key, int kernel, double gflops) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!db_) {
      Entry& e = mem_[key];
      e.kernel = kernel;
      e.gflops = gflops;
      return true;
    }
    const SqliteApi& s = sqlite_api();
    sqlite3_stmt* st = nullptr;
    if (s.prepare_v2(db_, "INSERT INTO kernel_cache(key_hash, best_kernel, best_gflops) VALUES(?1,?2,?3) "
                          "ON CONFLICT(key_hash) DO UPDATE SET best_kernel=excluded.best_kernel, "
                          "best_gflops=excluded.best_gflops;", -1, &st, nullptr) != kSqliteOk)
      return false;
    s.bind_text(st, 1, key.c_str(), -1, SF_SQLITE_TRANSIENT);
    s.bind_int(st, 2, kernel);
    s.bind_double(st, 3, gflops);
    const bool ok = s.step(st) == kSqliteDone;
    s.finalize(st);
    return ok;
  }

  bool mark_failed(const std::string& key, int code) {
    std::lock_guard<std::mutex> lk(mu_);
    if (!db_) {
      Entry& e = mem_[key];
      e.sparse_failed = 1;
      e.failure_count++;
      return true;
    }
    const SqliteApi& s = sqlite_api();
    sqlite3_stmt* st = nullptr;
    if (s.prepare_v2(db_, "INSERT INTO kernel_cache(key_hash, best_kernel, best_gflops, sparse_failed, "
                          "failure_count, last_failure_code, last_failure_ts) VALUES(?1,0,0,1,1,?2,?3) "
                          "ON CONFLICT(key_hash) DO UPDATE SET sparse_failed=1, "
                          "failure_count=failure_count+1, last_failure_code=?2, last_failure_ts=?3;",
                     -1, &st, nullptr) != kSqliteOk)
      return false;
    s.bind_text(st, 1, key.c_str(), -1, SF_SQLITE_TRANSIENT);
    s.bind_int(st, 2, code);
    s.bind_int64(st, 3, static_cast<long long>(time(nullptr)));
    const bool ok = s.step(st) == kSqliteDone;
    s.finalize(st);
    return ok;
  }

  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    mem_.clear();
    if (db_) exec("DELETE FROM kernel_cache;");
  }

  int size() {
    std::lock_guard<std::mutex> lk(mu_);
    if (!db_) return static_cast<int>(mem_.size());
    const SqliteApi& s = sqlite_api();
    sqlite3_stmt* st = nullptr;
    int n = 0;
    if (s.prepare_v2(db_, "SELECT COUNT(*) FROM kernel_cache;", -1, &st, nullptr) != kSqliteOk) return 0;
    if (s.step(st) == kSqliteRow) n = s.column_int(st, 0);
    s.finalize(st);
    return n;
  }

  bool persistent() const { return db_ != nullptr; }

 private:
  void exec(const char* sql) {
    char* err = nullptr;
    if (sqlite_api().exec(db_, sql, nullptr, nullptr, &err) != kSqliteOk) {
      SF_LOG("sqlite: %s", err ? err : "error");
      if (err) sqlite_api().free(err);
    }
  }
  bool has_column(const char* col) {
    const SqliteApi& s = sqlite_api();
    sqlite3_stmt* st = nullptr;
    std::string q = std::string("SELECT COUNT(*) FROM pragma_table_info('kernel_cache') WHERE name='") + col + "';";
    if (s.prepare_v2(db_, q.c_str(), -1, &st, nullptr) != kSqliteOk) return true;
    int n = 1;
    if (s.step(st) == kSqliteRow) n = s.column_int(st, 0);
    s.finalize(st);
    return n > 0;
  }
  std::string path_;
  sqlite3* db_ = nullptr;
  std::map<std::string, Entry> mem_;
  std::mutex mu_;
};

// ---------------------------------------------------------------- cuBLAS (dense candidate) via dlopen
struct CublasApi {
  int (*create)(void**);
  int (*destroy)(void*);
  int (*set_stream)(void*, cudaStream_t);
  int (*gemm_ex)(void*, int, int, int, int, int, const void*, const void*, int, int, const void*, int,
                 int, const void*, void*, int, int, int, int);
  bool ok = false;
};
const CublasApi& cublas_api() {
  static CublasApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libcublas.so.12", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libcublas.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    api.create = reinterpret_cast<decltype(api.create)>(dlsym(h, "cublasCreate_v2"));
    api.destroy = reinterpret_cast<decltype(api.destroy)>(dlsym(h, "cublasDestroy_v2"));
    api.set_stream = reinterpret_cast<decltype(api.set_stream)>(dlsym(h, "cublasSetStream_v2"));
    api.gemm_ex = reinterpret_cast<decltype(api.gemm_ex)>(dlsym(h, "cublasGemmEx"));
    api.ok = api.create && api.destroy && api.set_stream && api.gemm_ex;
  });
  return api;
}

// ---------------------------------------------------------------- selection
int bucket(int dim) {
  if (dim <= 0) return 0;
  uint32_t x = dim <= 32 ? 32u : static_cast<uint32_t>(dim);
  uint32_t p = 32;
  while (p < x && p < 65536u) p <<= 1;
  return p > 65535u ? 65535 : static_cast<int>(p);
}

std::string make_key(const sf_matmul_desc& d, int sm_arch) {
  char buf[160];
  snprintf(buf, sizeof(buf), "M=%d;N=%d;K=%d;dtype=%d;layout=%d;sp=%d;sm=%d", bucket(d.M), bucket(d.N),
           bucket(d.K), d.dtype & 0xFF, 0, d.sparsity_type & 0xFF, sm_arch & 0xFF);
  return buf;
}

std::string compressed_key(const sf_matmul_desc& d) {
  char buf[96];
  snprintf(buf, sizeof(buf), "%d/%d/%d/%d/%d", d.M, d.N, d.K, d.dtype, d.sparsity_type);
  return buf;
}

constexpr double kMinSparseFlops = 512.0 * 512.0 * 512.0;
constexpr int kMaxFailures = 3;
enum KernelId { kDenseTc = 0, kHybrid = 1, kSparsePrefill = 2, kSparseSmallM = 3 };

struct Timing {
  double mean_ms = -1;
  double cv = 0;
};

// ---------------------------------------------------------------- compressed-weight store
// Process-wide, keyed by content: FNV-1a 64 of the first KiB of the DEVICE matrix plus the shape, as
// upstream (cache/compressed_cache.cpp:9-29, compressed_cache.h:10-21 -- whose key narrows M, N, K to
// 16 bits; full ints here).  Values are library-owned device buffers in the layout the sparse GEMM
// consumes; entries are never evicted, and a put that would exceed 1 GiB is refused
// (compressed_cache.cpp:42,70-74).
uint64_t device_matrix_hash(const void* d_data, size_t bytes) {
  unsigned char sample[1024];
  const size_t n = bytes < sizeof(sample) ? bytes : sizeof(sample);
  if (n == 0 || cudaMemcpy(sample, d_data, n, cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  uint64_t h = 14695981039346656037ull;
  for (size_t i = 0; i < n; ++i) {
    h ^= sample[i];
    h *= 1099511628211ull;
  }
  return h;
}

struct CompressedKey {
  uint64_t content_hash;
  int32_t M, N, K, dtype, sparsity_type, device;
  bool operator<(const CompressedKey& o) const {
    return std::tie(content_hash, M, N, K, dtype, sparsity_type, device) <
           std::tie(o.content_hash, o.M, o.N, o.K, o.dtype, o.sparsity_type, o.device);
  }
};
struct CompressedValue {
  void* values = nullptr;
  void* meta = nullptr;
  size_t bytes = 0;
};
class CompressedStore {
 public:
  static constexpr size_t kMaxBytes = 1ull << 30;
  bool contains(const CompressedKey& k) {
    std::lock_guard<std::mutex> lk(mu_);
    return map_.count(k) != 0;
  }
  bool get(const CompressedKey& k, CompressedValue* out) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = map_.find(k);
    if (it == map_.end()) return false;
    *out = it->second;
    return true;
  }
  // Takes ownership of v's buffers on success; on refusal (cap) the caller frees them.
  bool put(const CompressedKey& k, const CompressedValue& v) {
    std::lock_guard<std::mutex> lk(mu_);
    if (map_.count(k)) return false;
    if (total_ + v.bytes > kMaxBytes) return false;
    map_[k] = v;
    total_ += v.bytes;
    return true;
  }
  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : map_) {
      int prev = 0;
      cudaGetDevice(&prev);
      cudaSetDevice(kv.first.device);
      cudaFree(kv.second.values);
      cudaFree(kv.second.meta);
      cudaSetDevice(prev);
    }
    map_.clear();
    total_ = 0;
  }
  size_t count() {
    std::lock_guard<std::mutex> lk(mu_);
    return map_.size();
  }
  size_t bytes() {
    std::lock_guard<std::mutex> lk(mu_);
    return total_;
  }
 private:
  std::mutex mu_;
  std::map<CompressedKey, CompressedValue> map_;
  size_t total_ = 0;
};
CompressedStore& compressed_store() {
  static CompressedStore* s = new CompressedStore;   // never destroyed: device buffers outlive static teardown
  return *s;
}

bool make_compressed_key(const sf_matmul_desc& d, const void* d_weight, CompressedKey* k) {
  if (!d_weight || d.M <= 0 || d.K <= 0) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const size_t bytes = static_cast<size_t>(d.M) * d.K * (d.dtype == 2 ? 4 : 2);
  const uint64_t h = device_matrix_hash(d_weight, bytes);
  if (h == 0) return false;
  *k = CompressedKey{h, d.M, d.N, d.K, d.dtype, d.sparsity_type, dev};
  return true;
}

int force_mode() {   // 0 none, 1 dense, 2 sparse
  const char* e = getenv("SPARSEFLOW_FORCE");
  if (!e || !*e) return 0;
  if (!strcmp(e, "dense") || !strcmp(e, "DENSE")) return 1;
  if (!strcmp(e, "sparse") || !strcmp(e, "SPARSE")) return 2;
  return 0;
}

// Decision counters of one selector (index = position in the array sf_get_counters fills).
enum Counter { kCtrCalls = 0, kCtrHits, kCtrMisses, kCtrBenchmarks, kCtrDense, kCtrSparse, kCtrFailures, kCtrForced, kNumCounters };

class Selector {
 public:
  explicit Selector(const std::string& path) : store_(path) {}

  // a, x, y: optional DEVICE matrices (weight [M, K], activations [N, K], output [N, M]); with a weight
  // the "compression cached" rule is evaluated on its content, and when all three are given the
  // candidates are timed on them instead of synthetic buffers.
  int select(const sf_matmul_desc& d, const sf_gpu_info& g, const void* a = nullptr, const void* x = nullptr,
             void* y = nullptr) {
    std::lock_guard<std::mutex> lk(mu_);
    ctr_[kCtrCalls]++;
    const std::string key = make_key(d, g.sm_arch);
    if (const int f = force_mode()) {
      ctr_[kCtrForced]++;
      const bool shape_ok = d.sparsity_type == 1 && (d.dtype == 0 || d.dtype == 1) && d.K % 64 == 0 && d.M % 8 == 0;
      const int k = (f == 2 && shape_ok) ? kSparsePrefill : kDenseTc;
      SF_LOG("SPARSEFLOW_FORCE: %s -> %d", key.c_str(), k);
      return k;
    }
    Entry e;
    if (store_.get(key, &e)) {
      if (e.failure_count > failures_[key]) failures_[key] = e.failure_count;
      // A row written only by a failure report (no measurement yet) must not pin the shape to dense:
      // below the quarantine threshold it is measured like a miss.
      const bool failure_stub = e.sparse_failed && e.kernel == kDenseTc && e.gflops == 0 && failures_[key] < kMaxFailures;
      if (!failure_stub) {
        ctr_[kCtrHits]++;
        SF_LOG("cache hit %s -> %d (%.1f GFLOPS)", key.c_str(), e.kernel, e.gflops);
        return e.kernel;
      }
    }
    ctr_[kCtrMisses]++;
    bool compression_cached = compressed_.count(compressed_key(d)) != 0;
    CompressedValue cv;
    if (a && d.sparsity_type == 1) {
      CompressedKey ck;
      if (make_compressed_key(d, a, &ck) && compressed_store().get(ck, &cv)) compression_cached = true;
    }
    std::string why;
    if (!eligible(d, key, compression_cached, &why)) {
      SF_LOG("sparse skipped for %s: %s; using dense", key.c_str(), why.c_str());
      store_.put_best(key, kDenseTc, 0.0);
      ctr_[kCtrDense]++;
      return kDenseTc;
    }
    double dense_ms = -1, sparse_ms = -1;
    ctr_[kCtrBenchmarks]++;
    const bool ran = benchmark(d, a, x, y, cv, &dense_ms, &sparse_ms);
    if (!ran) {
      SF_LOG("no device to benchmark on: dense, not cached");
      return kDenseTc;
    }
    if (sparse_ms <= 0) {
      failures_[key]++;
      ctr_[kCtrFailures]++;
      store_.mark_failed(key, -1);
    }
    int best = kDenseTc;
    double best_ms = dense_ms;
    if (sparse_ms > 0 && (dense_ms <= 0 || sparse_ms < dense_ms)) {
      best = d.N <= 8 ? kSparseSmallM : kSparsePrefill;
      best_ms = sparse_ms;
    }
    const double gflops = best_ms > 0 ? 2.0 * d.M * d.N * d.K / (best_ms * 1e6) : 0.0;
    SF_LOG("selected %d for %s: dense %.4f ms, sparse %.4f ms", best, key.c_str(), dense_ms, sparse_ms);
    store_.put_best(key, best, gflops);
    ctr_[best == kDenseTc ? kCtrDense : kCtrSparse]++;
    return best;
  }

  void note_compressed(const sf_matmul_desc& d) {
    std::lock_guard<std::mutex> lk(mu_);
    compressed_.insert(compressed_key(d));
  }
  void record_failure(const sf_matmul_desc& d, const sf_gpu_info& g) {
    std::lock_guard<std::mutex> lk(mu_);
    const std::string key = make_key(d, g.sm_arch);
    failures_[key]++;
    ctr_[kCtrFailures]++;
    store_.mark_failed(key, -1);
  }
  int size() { return store_.size(); }
  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    store_.clear();
    failures_.clear();
  }
  void counters(int64_t* out) {
    std::lock_guard<std::mutex> lk(mu_);
    for (int i = 0; i < kNumCounters; ++i) out[i] = ctr_[i];
  }

 private:
  bool eligible(const sf_matmul_desc& d, const std::string& key, bool compression_cached, std::string* why) {
    if (d.sparsity_type != 1) { *why = "Only 2:4 sparsity supported"; return false; }
    if (2.0 * d.M * d.N * d.K < kMinSparseFlops) { *why = "Matrix too small"; return false; }
    auto it = failures_.find(key);
    if (it != failures_.end() && it->second >= kMaxFailures) {
      *why = "Sparse failed too many times for this shape";
      return false;
    }
    if (!compression_cached) { *why = "Compression not cached, skipping sparse"; return false; }
    if (d.dtype != 0 && d.dtype != 1) { *why = "Only f16 / bf16 have a sparse kernel"; return false; }
    if (d.K % 64 != 0 || d.M % 8 != 0) { *why = "Shape not supported by the sparse kernel"; return false; }
    return true;
  }

  template <class F>
  Timing time_it(F&& launch, void* flush, size_t flush_bytes, cudaStream_t st) {
    Timing t;
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return t;
    auto run = [&](int iters) -> bool {
      std::vector<float> ms(iters);
      for (int i = 0; i < 3; ++i)
        if (!launch()) return false;
      for (int i = 0; i < iters; ++i) {
        cudaMemsetAsync(flush, i & 0xFF, flush_bytes, st);  // evict L2 between timed launches
        cudaEventRecord(e0, st);
        if (!launch()) return false;
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) return false;
        cudaEventElapsedTime(&ms[i], e0, e1);
      }
      double sum = 0, sq = 0;
      for (float v : ms) sum += v;
      const double mean = sum / iters;
      for (float v : ms) sq += (v - mean) * (v - mean);
      t.mean_ms = mean;
      t.cv = mean > 0 ? std::sqrt(sq / iters) / mean : 0;
      return true;
    };
    bool ok = run(10);
    if (ok && t.cv > 0.05) ok = run(20);
    if (!ok) t.mean_ms = -1;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return t;
  }

  // Weight = desc.M x desc.K (the sparse operand), activations = desc.N tokens.  Caller-provided
  // device matrices are used when all three are given (with the cached compressed form of the weight
  // when there is one); otherwise synthetic buffers, filled like the reference dispatcher's
  // (dispatch/kernel_dispatcher.cpp:105-131).
  bool benchmark(const sf_matmul_desc& d, const void* a_user, const void* x_user, void* y_user,
                 const CompressedValue& cached, double* dense_ms, double* sparse_ms) {
    int err = kOk;
    DeviceState* s = device_state(&err);
    if (!s) return false;
    const bool user = a_user && x_user && y_user;
    const size_t wb = static_cast<size_t>(d.M) * d.K * 2, xb = static_cast<size_t>(d.N) * d.K * 2,
                 yb = static_cast<size_t>(d.N) * d.M * 2, flush_bytes = 256u << 20;
    void *w = nullptr, *x = nullptr, *y = nullptr, *vals = nullptr, *meta = nullptr, *flush = nullptr;
    auto free_all = [&] {
      for (void* p : {w, x, y, vals, meta, flush})
        if (p) cudaFree(p);
    };
    bool alloc_ok = cudaMalloc(&flush, flush_bytes) == cudaSuccess;
    if (alloc_ok && !user)
      alloc_ok = cudaMalloc(&w, wb) == cudaSuccess && cudaMalloc(&x, xb) == cudaSuccess &&
                 cudaMalloc(&y, yb) == cudaSuccess;
    if (alloc_ok && !cached.values)
      alloc_ok = cudaMalloc(&vals, values_bytes(d.M, d.K)) == cudaSuccess &&
                 cudaMalloc(&meta, meta_bytes(d.M, d.K)) == cudaSuccess;
    if (!alloc_ok) {
      cudaGetLastError();
      free_all();
      return false;
    }
    if (!user) {  // weight pattern 1,1,0,0 ; activations 1.0
      const uint16_t one = d.dtype == 1 ? 0x3F80 : 0x3C00;
      std::vector<uint16_t> hw(static_cast<size_t>(d.M) * d.K), hx(static_cast<size_t>(d.N) * d.K, one);
      for (size_t i = 0; i < hw.size(); ++i) hw[i] = (i & 3) < 2 ? one : 0;
      cudaMemcpy(w, hw.data(), wb, cudaMemcpyHostToDevice);
      cudaMemcpy(x, hx.data(), xb, cudaMemcpyHostToDevice);
    }
    const void* wsrc = user ? a_user : w;
    const void* xsrc = user ? x_user : x;
    void* ydst = user ? y_user : y;
    cudaStream_t st = nullptr;
    bool sparse_ok = true;
    const void* use_vals = cached.values;
    const void* use_meta = cached.meta;
    if (!use_vals) {
      PruneArgs pa{};
      pa.dense = wsrc; pa.rows = d.M; pa.K = d.K; pa.ld = d.K; pa.fmt = d.dtype; pa.tie = kTieHigh;
      pa.values = vals; pa.meta = meta;
      sparse_ok = launch_prune_compress(pa, st) == kOk;
      use_vals = vals;
      use_meta = meta;
    }
    SparseGemmArgs ga{};
    ga.x = xsrc; ga.values = use_vals; ga.meta = use_meta; ga.y = ydst; ga.status = s->status;
    ga.m_tok = d.N; ga.n_out = d.M; ga.K = d.K; ga.ldx = d.K; ga.ldy = d.M; ga.fmt = d.dtype;
    ga.epi = kEpiStore; ga.act = kActNone; ga.num_sms = s->num_sms;
    if (sparse_ok) {
      Timing ts = time_it([&] { return launch_sparse_gemm(ga, st) == kOk; }, flush, flush_bytes, st);
      int word = 0;
      cudaMemcpy(&word, s->status, sizeof(int), cudaMemcpyDeviceToHost);
      if (word != 0) {
        cudaMemset(s->status, 0, sizeof(int));
        ts.mean_ms = -1;
      }
      *sparse_ms = ts.mean_ms;
    }
    const CublasApi& cb = cublas_api();
    if (cb.ok) {
      void* h = nullptr;
      if (cb.create(&h) == 0) {
        cb.set_stream(h, st);
        const float alpha = 1.f, beta = 0.f;
        const int dt = d.dtype == 1 ? 14 /*CUDA_R_16BF*/ : 2 /*CUDA_R_16F*/;
        // row-major Y[N,M] = X[N,K] . W[M,K]^T  ==  column-major Y^T[M,N] = W^T(op T) . X
        Timing td = time_it(
            [&] {
              return cb.gemm_ex(h, 1 /*T*/, 0 /*N*/, d.M, d.N, d.K, &alpha, wsrc, dt, d.K, xsrc, dt, d.K, &beta,
                                ydst, dt, d.M, 68 /*CUBLAS_COMPUTE_32F*/, -1 /*default algo*/) == 0;
            },
            flush, flush_bytes, st);
        *dense_ms = td.mean_ms;
        cb.destroy(h);
      }
    }
    cudaDeviceSynchronize();
    free_all();
    return true;
  }

  KernelStore store_;
  std::mutex mu_;
  std::map<std::string, int> failures_;
  std::set<std::string> compressed_;
  int64_t ctr_[kNumCounters] = {};
};

std::mutex g_mu;
std::map<std::string, std::unique_ptr<Selector>> g_selectors;

std::string resolve_path(const char* cache_path) {
  if (cache_path) return cache_path;
  const char* e = getenv("SPARSEFLOW_CACHE_DB");
  return (e && *e) ? e : "kernel_cache.db";
}

Selector* selector_for(const char* cache_path) {
  const std::string path = resolve_path(cache_path);
  std::lock_guard<std::mutex> lk(g_mu);
  auto& p = g_selectors[path];
  if (!p) p.reset(new Selector(path));
  return p.get();
}

}  // namespace
}  // namespace sfb200

using namespace sfb200;

extern "C" {

int32_t sf_select_kernel(const char* cache_path, const sf_matmul_desc* desc, const sf_gpu_info* gpu) {
  if (!desc || !gpu) return 0;
  return selector_for(cache_path)->select(*desc, *gpu);
}

// Both go through the process's selector for that path, so the in-memory store (used when
// libsqlite3 is absent) and the failure counts are covered too.
int32_t sf_cache_size(const char* cache_path) { return selector_for(cache_path)->size(); }

void sf_cache_clear(const char* cache_path) { selector_for(cache_path)->clear(); }

int32_t sf_select_kernel_ex(const char* cache_path, const sf_matmul_desc* desc, const sf_gpu_info* gpu,
                            const void* d_weight, const void* d_x, void* d_y) {
  if (!desc || !gpu) return 0;
  return selector_for(cache_path)->select(*desc, *gpu, d_weight, d_x, d_y);
}

int32_t sf_compress_weight(const sf_matmul_desc* desc, const void* d_weight, const void** values,
                           const void** meta) {
  if (values) *values = nullptr;
  if (meta) *meta = nullptr;
  if (!desc || !d_weight || desc->sparsity_type != 1 || (desc->dtype != 0 && desc->dtype != 1)) return 0;
  if (desc->M <= 0 || desc->K <= 0 || desc->K % 16 != 0) return 0;
  int err = kOk;
  if (!device_state(&err)) return 0;
  CompressedKey key;
  if (!make_compressed_key(*desc, d_weight, &key)) return 0;
  CompressedValue v;
  if (compressed_store().get(key, &v)) {
    if (values) *values = v.values;
    if (meta) *meta = v.meta;
    return 1;
  }
  const size_t vb = values_bytes(desc->M, desc->K), mb = meta_bytes(desc->M, desc->K);
  if (compressed_store().bytes() + vb + mb > CompressedStore::kMaxBytes) return 0;
  if (cudaMalloc(&v.values, vb) != cudaSuccess || cudaMalloc(&v.meta, mb) != cudaSuccess) {
    cudaGetLastError();
    if (v.values) cudaFree(v.values);
    return 0;
  }
  v.bytes = vb + mb;
  PruneArgs pa{};
  pa.dense = d_weight; pa.rows = desc->M; pa.K = desc->K; pa.ld = desc->K; pa.fmt = desc->dtype; pa.tie = kTieHigh;
  pa.values = v.values; pa.meta = v.meta;
  const bool ok = launch_prune_compress(pa, nullptr) == kOk && cudaStreamSynchronize(nullptr) == cudaSuccess &&
                  compressed_store().put(key, v);
  if (!ok) {
    cudaFree(v.values);
    cudaFree(v.meta);
    return 0;
  }
  if (values) *values = v.values;
  if (meta) *meta = v.meta;
  return 1;
}

int32_t sf_compressed_cache_count(void) { return static_cast<int32_t>(compressed_store().count()); }
uint64_t sf_compressed_cache_bytes(void) { return compressed_store().bytes(); }
void sf_compressed_cache_clear(void) { compressed_store().clear(); }

int32_t sf_get_counters(const char* cache_path, int64_t* out, int32_t n) {
  if (!out || n <= 0) return 0;
  int64_t c[kNumCounters];
  selector_for(cache_path)->counters(c);
  const int m = n < kNumCounters ? n : kNumCounters;
  for (int i = 0; i < m; ++i) out[i] = c[i];
  return m;
}

void sf_note_compressed(const char* cache_path, const sf_matmul_desc* desc) {
  if (desc) selector_for(cache_path)->note_compressed(*desc);
}

void sf_record_sparse_failure(const char* cache_path, const sf_matmul_desc* desc, const sf_gpu_info* gpu) {
  if (desc && gpu) selector_for(cache_path)->record_failure(*desc, *gpu);
}

int32_t sf_bucket_dimension(int32_t dim) { return bucket(dim); }

}  // extern "C"
