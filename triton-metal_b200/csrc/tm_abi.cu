// The tm_* C ABI of libtmcuda: handle table, error slot, buffers, descriptor
// "libraries", and launch marshalling.  Mirrors the behaviour of the reference's
// exports (Sources/TritonMetalCore/Compiler.swift:172-479 and
// Sources/TritonMetalCore/Runtime.swift:250-321) over the CUDA runtime.

#include "../../include/tm.h"
#include "tm_core.h"
#include "attn_schedule.h"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

using namespace tmc;

namespace {

// ---------------------------------------------------------------------------
// Last-error slot: one per process, lock protected, cleared by tm_last_error
// (Compiler.swift:461-479).
// ---------------------------------------------------------------------------
std::mutex g_error_lock;
std::string g_error;
bool g_has_error = false;

void store_error(const std::string& message) {
  std::lock_guard<std::mutex> guard(g_error_lock);
  g_error = message;
  g_has_error = true;
}

char* dup_string(const std::string& s) {
  char* out = (char*)std::malloc(s.size() + 1);
  if (out) std::memcpy(out, s.c_str(), s.size() + 1);
  return out;
}

std::string invalid_argument(const std::string& m) { return "invalid argument: " + m; }
std::string invalid_handle(const std::string& m) { return "invalid handle: " + m; }
std::string cuda_error(const std::string& m) { return "metal error: " + m; }  // CoreError.metal wording

// ---------------------------------------------------------------------------
// Objects behind handles
// ---------------------------------------------------------------------------
enum class ObjKind { Library, Kernel, Buffer };

struct Object {
  ObjKind kind;
  virtual ~Object() {}
  explicit Object(ObjKind k) : kind(k) {}
};

struct LibraryObj : Object {
  std::vector<KernelDesc> kernels;
  // A binary image (cubin / fatbin) handed to tm_load_metallib: the caller's own kernels, loaded
  // as they are.  The bytes are kept for as long as the image is.
  std::string image_bytes;
  cudaLibrary_t image = nullptr;
  LibraryObj() : Object(ObjKind::Library) {}
  ~LibraryObj() override {
    if (image) cudaLibraryUnload(image);
  }
};

struct KernelObj : Object {
  KernelDesc desc;
  int path_option = 0;   // 0 auto, 1 SIMT, 2 tcgen05 required
  int last_path = 0;
  // Entry point of a binary image (null for the library's own kernels): its name, the size of
  // every parameter as the image declares them, and the image itself, kept loaded.
  cudaKernel_t binary = nullptr;
  std::string binary_name;
  std::vector<size_t> param_sizes;
  int max_threads = 1024;
  std::shared_ptr<LibraryObj> owner;
  KernelObj() : Object(ObjKind::Kernel) {}
};

struct BufferObj : Object {
  void* ptr = nullptr;
  int64_t length = 0;
  bool host_exposed = false;   // tm_buffer_contents handed the pointer to the host
  bool device_only = false;    // plain device memory (tmx_alloc_device_buffer): no host pointer
  bool imported = false;       // another process's device memory, mapped by tmx_ipc_import
  // Ordering of tmx_buffer_write_async (which runs on a stream of its own) against the rest:
  uint64_t last_launch = 0;    // number of the last launch that took this buffer as an argument
  bool read_async_since_write = false;   // a tmx_buffer_read_async of it may still be in flight
  BufferObj() : Object(ObjKind::Buffer) {}
  ~BufferObj() override {
    if (!ptr) return;
    if (imported) cudaIpcCloseMemHandle(ptr);
    else cudaFree(ptr);
  }
};

const char* kind_word(ObjKind k) {
  return k == ObjKind::Library ? "library" : (k == ObjKind::Kernel ? "kernel" : "buffer");
}

// One process-wide table; handle 0 is never valid; first handle is 1
// (Runtime.swift:250-290).
class HandleTable {
 public:
  int64_t insert(std::shared_ptr<Object> obj) {
    std::lock_guard<std::mutex> guard(lock_);
    int64_t h = next_++;
    table_[h] = std::move(obj);
    return h;
  }
  // Typed lookup with the reference's two messages.
  std::shared_ptr<Object> lookup(int64_t handle, ObjKind kind, std::string& err) {
    std::lock_guard<std::mutex> guard(lock_);
    auto it = table_.find(handle);
    if (it == table_.end()) {
      err = invalid_handle(std::string(kind_word(kind)) + " handle " + std::to_string(handle) +
                           " is not live");
      return nullptr;
    }
    if (it->second->kind != kind) {
      err = invalid_handle("handle " + std::to_string(handle) + " is not a " + kind_word(kind));
      return nullptr;
    }
    return it->second;
  }
  bool remove(int64_t handle) {
    std::shared_ptr<Object> victim;   // destroyed outside the lock
    {
      std::lock_guard<std::mutex> guard(lock_);
      auto it = table_.find(handle);
      if (it == table_.end()) return false;
      victim = std::move(it->second);
      table_.erase(it);
    }
    return true;
  }
  int64_t count() {
    std::lock_guard<std::mutex> guard(lock_);
    return (int64_t)table_.size();
  }

 private:
  std::mutex lock_;
  std::map<int64_t, std::shared_ptr<Object>> table_;
  int64_t next_ = 1;
};

HandleTable g_handles;

template <class T>
std::shared_ptr<T> lookup_as(int64_t handle, ObjKind kind, std::string& err) {
  return std::static_pointer_cast<T>(g_handles.lookup(handle, kind, err));
}

// ---------------------------------------------------------------------------
// Device context: one device, one stream per process (Runtime.swift:10-11)
// ---------------------------------------------------------------------------
struct Device {
  std::mutex lock;
  bool tried = false;
  bool ok = false;
  std::string why;           // why not ok
  int ordinal = -1;          // -1: take $TMCUDA_DEVICE or 0
  int count = 0;
  cudaDeviceProp prop{};
  cudaStream_t stream = nullptr;
  // device -> host copies of tmx_buffer_read_async run here, behind an event on `stream`, so
  // that they overlap the host -> device copies and kernels enqueued after them
  cudaStream_t read_stream = nullptr;
  cudaEvent_t ev_read = nullptr, ev_join = nullptr;
  bool reads_in_flight = false;
  // Host -> device copies of tmx_buffer_write_async run on a third stream, so that the upload
  // of the next piece of input overlaps the kernels enqueued before it (on `stream` the copy
  // would wait for them).  Stream order is kept per buffer: the copy waits for the last launch
  // that took the buffer (every launch records an event once asynchronous writes are in use;
  // the last kEventRing of them are kept) and for a read-back of it still in flight, and
  // `stream` waits for the copy, so everything enqueued afterwards sees the new contents.
  static constexpr int kEventRing = 64;
  cudaStream_t write_stream = nullptr;
  cudaEvent_t launch_events[kEventRing] = {};
  uint64_t launch_event_number[kEventRing] = {};
  cudaEvent_t write_events[kEventRing] = {};
  cudaEvent_t ev_order = nullptr;
  uint64_t launch_number = 0, write_number = 0;
  bool async_writes = false;
  std::vector<std::weak_ptr<BufferObj>> read_back;   // buffers with a read-back possibly in flight
  std::recursive_mutex order_lock;   // guards the ordering state above (callers may be threads)
  DeviceStatus* status = nullptr;   // pinned, device-visible
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  // capability probe
  bool probed = false;
  std::string unusable;      // empty when usable
  int64_t launches = 0;
  unsigned int* gather_counter = nullptr;   // device word: CTAs of a gathered GEMM that are done
};

Device g_dev;

bool ensure_device(std::string& err) {
  std::lock_guard<std::mutex> guard(g_dev.lock);
  if (g_dev.tried) {
    if (!g_dev.ok) err = g_dev.why;
    return g_dev.ok;
  }
  g_dev.tried = true;
  auto fail = [&](const std::string& m) {
    g_dev.why = cuda_error(m);
    err = g_dev.why;
    return false;
  };
  cudaError_t e = cudaGetDeviceCount(&g_dev.count);
  if (e != cudaSuccess || g_dev.count == 0) {
    cudaGetLastError();
    return fail("no CUDA device available on this system");
  }
  if (g_dev.ordinal < 0) {
    const char* env = std::getenv("TMCUDA_DEVICE");
    g_dev.ordinal = env ? std::atoi(env) : 0;
  }
  if (g_dev.ordinal >= g_dev.count)
    return fail("device ordinal " + std::to_string(g_dev.ordinal) + " out of range (" +
                std::to_string(g_dev.count) + " devices)");
  if ((e = cudaSetDevice(g_dev.ordinal)) != cudaSuccess)
    return fail(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  if ((e = cudaGetDeviceProperties(&g_dev.prop, g_dev.ordinal)) != cudaSuccess)
    return fail(std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
  if ((e = cudaStreamCreateWithFlags(&g_dev.stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail(std::string("could not create a CUDA stream: ") + cudaGetErrorString(e));
  if ((e = cudaHostAlloc((void**)&g_dev.status, sizeof(DeviceStatus), cudaHostAllocMapped)) !=
      cudaSuccess)
    return fail(std::string("could not allocate the status word: ") + cudaGetErrorString(e));
  std::memset(g_dev.status, 0, sizeof(DeviceStatus));
  cudaEventCreate(&g_dev.ev_begin);
  cudaEventCreate(&g_dev.ev_end);
  if ((e = cudaStreamCreateWithFlags(&g_dev.read_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail(std::string("could not create the read-back stream: ") + cudaGetErrorString(e));
  cudaEventCreateWithFlags(&g_dev.ev_read, cudaEventDisableTiming);
  cudaEventCreateWithFlags(&g_dev.ev_join, cudaEventDisableTiming);
  if ((e = cudaStreamCreateWithFlags(&g_dev.write_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail(std::string("could not create the upload stream: ") + cudaGetErrorString(e));
  cudaEventCreateWithFlags(&g_dev.ev_order, cudaEventDisableTiming);
  for (int i = 0; i < Device::kEventRing; ++i) {
    cudaEventCreateWithFlags(&g_dev.launch_events[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&g_dev.write_events[i], cudaEventDisableTiming);
  }
  g_dev.ok = true;
  return true;
}

// The calling thread must have the library's device current before any CUDA call.
bool bind_device(std::string& err) {
  if (!ensure_device(err)) return false;
  cudaSetDevice(g_dev.ordinal);
  return true;
}

LaunchCtx launch_ctx() {
  LaunchCtx c;
  c.stream = g_dev.stream;
  c.sm_count = g_dev.prop.multiProcessorCount;
  c.status = g_dev.status;
  c.launches = &g_dev.launches;
  return c;
}

// Capability probe, once per process (Runtime.swift:125-178): the device must be
// compute capability 10.x and run a kernel of this library that stores a value.
const std::string& unusable_reason() {
  std::string err;
  if (!bind_device(err)) {
    static std::string none;
    none = err.rfind("metal error: ", 0) == 0 ? err.substr(13) : err;
    return none;
  }
  std::lock_guard<std::mutex> guard(g_dev.lock);
  if (g_dev.probed) return g_dev.unusable;
  g_dev.probed = true;
  if (g_dev.prop.major != 10) {
    g_dev.unusable = std::string("device '") + g_dev.prop.name + "' is sm_" +
                     std::to_string(g_dev.prop.major) + std::to_string(g_dev.prop.minor) +
                     "; libtmcuda holds sm_100a code only";
    return g_dev.unusable;
  }
  int got = 0;
  std::string e = launch_probe(launch_ctx(), &got);
  if (!e.empty()) g_dev.unusable = "probe kernel failed: " + e;
  else if (got != 0x7a11) g_dev.unusable = "probe kernel stored the wrong value";
  return g_dev.unusable;
}

// Wait for the stream and surface device-side status.
// Make the library's stream wait for the read-backs enqueued on the side stream.
// (Every caller synchronises the library's stream right afterwards, so the read-backs are
// complete when it returns and the buffers' marks can go.)
void join_reads() {
  std::lock_guard<std::recursive_mutex> guard(g_dev.order_lock);
  if (!g_dev.reads_in_flight) return;
  cudaEventRecord(g_dev.ev_join, g_dev.read_stream);
  cudaStreamWaitEvent(g_dev.stream, g_dev.ev_join, 0);
  g_dev.reads_in_flight = false;
  for (auto& weak : g_dev.read_back)
    if (auto b = weak.lock()) b->read_async_since_write = false;
  g_dev.read_back.clear();
}

bool sync_stream(std::string& err) {
  join_reads();
  cudaError_t e = cudaStreamSynchronize(g_dev.stream);
  if (e != cudaSuccess) {
    err = cuda_error(std::string("kernel execution failed: ") + cudaGetErrorString(e));
    return false;
  }
  if (g_dev.status->code != 0) {
    DeviceStatus s = *g_dev.status;
    std::memset(g_dev.status, 0, sizeof(DeviceStatus));
    err = cuda_error("kernel execution failed: a bounded wait gave up inside the kernel (code " +
                     std::to_string(s.code) + ", site " + std::to_string(s.where) + ", block " +
                     std::to_string(s.block) + ", detail " + std::to_string(s.extra) +
                     "); the results of this launch are not valid");
    return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// Launch marshalling
// ---------------------------------------------------------------------------
struct Decoded {
  std::map<int, std::shared_ptr<BufferObj>> buffers;   // by Role
  std::map<int, int64_t> ints;
  std::map<int, float> floats;
  float sm_scale = 0.f;
};

bool decode_args(KernelObj& k, const int32_t* kinds, const int64_t* values, int32_t argc,
                 Decoded& out, std::string& err) {
  if (argc > 0 && (!kinds || !values)) {
    err = invalid_argument("tm_launch received NULL argument arrays");
    return false;
  }
  // Kinds are validated for every position first, as the reference does while
  // it builds its argument list (Compiler.swift:419-436).
  for (int i = 0; i < argc; ++i) {
    if (kinds[i] < 0 || kinds[i] > 3) {
      err = invalid_argument("unknown launch argument kind " + std::to_string(kinds[i]) +
                             " at position " + std::to_string(i));
      return false;
    }
  }
  const auto& args = k.desc.args;
  if (argc != (int)args.size()) {
    err = invalid_argument(std::string(kernel_entry_name(k.desc.id)) + " takes " +
                           std::to_string(args.size()) + " arguments, tm_launch received " +
                           std::to_string(argc));
    return false;
  }
  for (int i = 0; i < argc; ++i) {
    const ArgInfo& a = args[i];
    if (a.is_pointer) {
      if (kinds[i] != 0) {
        err = invalid_argument("argument " + std::to_string(i) + " of " +
                               kernel_entry_name(k.desc.id) + " is a pointer; expected kind 0, got " +
                               std::to_string(kinds[i]));
        return false;
      }
      auto b = lookup_as<BufferObj>(values[i], ObjKind::Buffer, err);
      if (!b) return false;
      out.buffers[(int)a.role] = b;
    } else if (a.dtype == "f32") {
      if (kinds[i] != 2) {
        err = invalid_argument("argument " + std::to_string(i) + " of " +
                               kernel_entry_name(k.desc.id) + " is an f32 scalar; expected kind 2, got " +
                               std::to_string(kinds[i]));
        return false;
      }
      uint32_t bits = (uint32_t)(values[i] & 0xffffffffu);
      float f;
      std::memcpy(&f, &bits, 4);
      if (a.role == Role::SmScale) out.sm_scale = f;
      out.floats[(int)a.role] = f;
    } else {
      if (kinds[i] != 1 && kinds[i] != 3) {
        err = invalid_argument("argument " + std::to_string(i) + " of " +
                               kernel_entry_name(k.desc.id) +
                               " is an integer scalar; expected kind 1 or 3, got " +
                               std::to_string(kinds[i]));
        return false;
      }
      int64_t v = kinds[i] == 1 ? (int64_t)(int32_t)(values[i] & 0xffffffff) : values[i];
      out.ints[(int)a.role] = v;
    }
  }
  return true;
}

// One dimension of the region a kernel addresses: `count` elements `stride` apart.
struct Span {
  int64_t count, stride;
};

// Refuses a launch whose largest element index - the sum of (count - 1) * stride over the
// dimensions - lies beyond the buffer.  The index is formed in 128 bits from its factors, so
// an absurd extent or stride cannot wrap into something that looks in bounds.
bool check_extent(const BufferObj& b, std::initializer_list<Span> dims, int elt_bytes, const char* what,
                  std::string& err) {
  __int128 last = 0;
  for (const Span& d : dims) {
    if (d.count <= 0) return true;      // an empty dimension: nothing is addressed
    last += ((__int128)d.count - 1) * (__int128)d.stride;
  }
  const __int128 need = (last + 1) * elt_bytes;
  if (need > (__int128)b.length) {
    // the byte count is printed when it fits 64 bits, else as "more than 2^63"
    const std::string shown = need < ((__int128)1 << 63) ? std::to_string((long long)need) : "more than 2^63";
    err = invalid_argument(std::string("launch would address ") + shown + " bytes of " + what +
                           ", beyond its " + std::to_string(b.length) + "-byte buffer");
    return false;
  }
  return true;
}

// Extents the kernels index with 32-bit integers.
bool check_int32(int64_t v, const char* name, std::string& err) {
  if (v > 0x7fffffffll) {
    err = invalid_argument(std::string(name) + " " + std::to_string(v) + " is above 2^31 - 1");
    return false;
  }
  return true;
}

int64_t get_int(const Decoded& d, Role r, int64_t fallback) {
  auto it = d.ints.find((int)r);
  return it == d.ints.end() ? fallback : it->second;
}

void prefetch_exposed(const Decoded& d) {
  // Buffers whose host pointer was handed out may have migrated to the host;
  // bring them back before the kernel touches them (the migration is not part of
  // any timed region: benchmarks never expose their buffers).
  for (auto& kv : d.buffers) {
    if (kv.second->host_exposed)
      cudaMemPrefetchAsync(kv.second->ptr, (size_t)kv.second->length, g_dev.ordinal, g_dev.stream);
  }
}

// Enqueue one launch (no wait).  Returns false with `err` on failure.
// Called once a launch is on the stream: numbers it, remembers the number in every buffer it
// took, and - once tmx_buffer_write_async is in use - records the event a later asynchronous
// write into one of those buffers will wait for.
template <typename Buffers>
void note_launch(const Buffers& buffers) {
  std::lock_guard<std::recursive_mutex> guard(g_dev.order_lock);
  const uint64_t n = ++g_dev.launch_number;
  for (BufferObj* b : buffers)
    if (b) b->last_launch = n;
  if (g_dev.async_writes) {
    const int slot = (int)(n % Device::kEventRing);
    cudaEventRecord(g_dev.launch_events[slot], g_dev.stream);
    g_dev.launch_event_number[slot] = n;
  }
}

// A kernel of a binary image: the arguments go to the entry point in the order given, a buffer
// as its device address, scalars in their own width (Runtime.swift:213-231 binds them the same
// way: argument i at index i).  Count and widths are checked against what the image declares,
// so that a mismatched call is an error message and not a fault on the device.
bool enqueue_binary(KernelObj& k, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
                    const int32_t* kinds, const int64_t* values, int32_t argc, int repeats,
                    std::string& err) {
  if (argc > 0 && (!kinds || !values)) {
    err = invalid_argument("tm_launch received NULL argument arrays");
    return false;
  }
  if (gx <= 0 || gy <= 0 || gz <= 0) {
    err = invalid_argument("threadgroup grid must be positive in every dimension");
    return false;
  }
  if (threads <= 0) {
    err = invalid_argument("threadsPerThreadgroup must be positive");
    return false;
  }
  if (threads > k.max_threads) {
    err = invalid_argument("threadsPerThreadgroup " + std::to_string(threads) +
                           " exceeds the pipeline maximum " + std::to_string(k.max_threads));
    return false;
  }
  if (gx > 0x7fffffffll || gy > 65535 || gz > 65535) {
    err = invalid_argument("threadgroup grid exceeds what the device can launch");
    return false;
  }
  if ((size_t)argc != k.param_sizes.size()) {
    err = invalid_argument("kernel '" + k.binary_name + "' takes " + std::to_string(k.param_sizes.size()) +
                           " arguments, got " + std::to_string(argc));
    return false;
  }
  std::vector<uint64_t> storage((size_t)argc);
  std::vector<void*> args((size_t)argc);
  std::vector<std::shared_ptr<BufferObj>> buffers;
  for (int i = 0; i < argc; ++i) {
    size_t width = 0;
    switch (kinds[i]) {
      case 0: {
        auto b = lookup_as<BufferObj>(values[i], ObjKind::Buffer, err);
        if (!b) return false;
        storage[i] = (uint64_t)(uintptr_t)b->ptr;
        buffers.push_back(b);
        width = 8;
        break;
      }
      case 1: storage[i] = (uint32_t)values[i]; width = 4; break;
      case 2: storage[i] = (uint32_t)values[i]; width = 4; break;
      case 3: storage[i] = (uint64_t)values[i]; width = 8; break;
      default:
        err = invalid_argument("unknown launch argument kind " + std::to_string(kinds[i]) + " at position " +
                               std::to_string(i));
        return false;
    }
    if (k.param_sizes[i] != width) {
      err = invalid_argument("argument " + std::to_string(i) + " of kernel '" + k.binary_name + "' is " +
                             std::to_string(k.param_sizes[i]) + " bytes wide, the launch passes " +
                             std::to_string(width));
      return false;
    }
    args[i] = &storage[i];
  }
  if (!bind_device(err)) return false;
  std::vector<BufferObj*> raw;
  bool waited = false;
  for (auto& b : buffers) {
    raw.push_back(b.get());
    if (b->host_exposed) cudaMemPrefetchAsync(b->ptr, (size_t)b->length, g_dev.ordinal, g_dev.stream);
    if (b->read_async_since_write && !waited) {
      cudaEventRecord(g_dev.ev_order, g_dev.read_stream);
      cudaStreamWaitEvent(g_dev.stream, g_dev.ev_order, 0);
      waited = true;
    }
  }
  for (int r = 0; r < repeats; ++r) {
    cudaError_t e = cudaLaunchKernel((const void*)k.binary, dim3((unsigned)gx, (unsigned)gy, (unsigned)gz),
                                     dim3((unsigned)threads, 1, 1), args.data(), 0, g_dev.stream);
    if (e != cudaSuccess) {
      cudaGetLastError();
      err = cuda_error("launch of '" + k.binary_name + "' failed: " + cudaGetErrorString(e));
      return false;
    }
    ++g_dev.launches;
  }
  k.last_path = 0;
  note_launch(raw);
  return true;
}

bool enqueue(KernelObj& k, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
             const int32_t* kinds, const int64_t* values, int32_t argc, int repeats,
             std::string& err) {
  if (k.binary) return enqueue_binary(k, gx, gy, gz, threads, kinds, values, argc, repeats, err);
  Decoded d;
  if (!decode_args(k, kinds, values, argc, d, err)) return false;
  struct NoteOnExit {
    Decoded& d;
    bool armed = false;
    ~NoteOnExit() {
      if (!armed) return;
      std::vector<BufferObj*> bufs;
      for (auto& kv : d.buffers) bufs.push_back(kv.second.get());
      note_launch(bufs);
    }
  } note{d};
  // Runtime.swift:201-211
  if (gx <= 0 || gy <= 0 || gz <= 0) {
    err = invalid_argument("threadgroup grid must be positive in every dimension");
    return false;
  }
  if (threads <= 0) {
    err = invalid_argument("threadsPerThreadgroup must be positive");
    return false;
  }
  if (threads > 1024) {
    err = invalid_argument("threadsPerThreadgroup " + std::to_string(threads) +
                           " exceeds the pipeline maximum 1024");
    return false;
  }
  if (!bind_device(err)) return false;
  {
    const std::string& why = unusable_reason();
    if (!why.empty()) {
      err = cuda_error(why);
      return false;
    }
  }
  // a buffer whose read-back may still be in flight must not be overwritten under it
  for (auto& kv : d.buffers) {
    if (kv.second && kv.second->read_async_since_write) {
      cudaEventRecord(g_dev.ev_order, g_dev.read_stream);
      cudaStreamWaitEvent(g_dev.stream, g_dev.ev_order, 0);
      break;
    }
  }
  LaunchCtx ctx = launch_ctx();
  const KernelDesc& desc = k.desc;
  const int eb = elt_size(desc.elt);
  auto buf = [&](Role r) -> BufferObj* {
    auto it = d.buffers.find((int)r);
    return it == d.buffers.end() ? nullptr : it->second.get();
  };
  auto nonneg = [&](int64_t v, const char* name) {
    if (v < 0) {
      err = invalid_argument(std::string(name) + " must not be negative, got " + std::to_string(v));
      return false;
    }
    return true;
  };

  if (is_rowwise(desc.id)) {
    // ---- one-dimensional kernels: program p covers [p*BLOCK, (p+1)*BLOCK) (rows for softmax) ----
    RowProblem p{};
    p.id = desc.id;
    BufferObj *in0 = buf(Role::In0), *in1 = buf(Role::In1), *outb = buf(Role::Out);
    if (!in0 || !outb || ((desc.id == KernelId::VecAdd || desc.id == KernelId::VecMul) && !in1)) {
      err = invalid_argument(std::string(kernel_entry_name(desc.id)) + " was loaded from a descriptor without its buffer arguments");
      return false;
    }
    p.in0 = (const float*)in0->ptr;
    p.in1 = in1 ? (const float*)in1->ptr : nullptr;
    p.out = (float*)outb->ptr;
    auto f = [&](Role r) {
      auto it = d.floats.find((int)r);
      return it == d.floats.end() ? 0.f : it->second;
    };
    p.scale = f(Role::Scale);
    p.bias = f(Role::Bias);
    const int64_t block = desc.block_m;
    if (desc.id == KernelId::Softmax) {
      p.rows = gx;
      p.cols = std::min<int64_t>(get_int(d, Role::NCols, 0), block);
      p.stride_in = get_int(d, Role::StrideIn, 0);
      p.stride_out = get_int(d, Role::StrideOut, 0);
      if (!nonneg(p.stride_in, "the input row stride") || !nonneg(p.stride_out, "the output row stride"))
        return false;
      if (p.cols <= 0) return true;
      if (!check_int32(p.rows, "the row count", err)) return false;
      if (!check_extent(*in0, {{p.rows, p.stride_in}, {p.cols, 1}}, 4, "the input", err)) return false;
      if (!check_extent(*outb, {{p.rows, p.stride_out}, {p.cols, 1}}, 4, "the output", err)) return false;
    } else {
      p.limit = std::min<int64_t>(get_int(d, Role::Count, 0), gx * block);
      if (p.limit <= 0) return true;
      if (!check_extent(*in0, {{p.limit, 1}}, 4, "the first input", err)) return false;
      if (in1 && !check_extent(*in1, {{p.limit, 1}}, 4, "the second input", err)) return false;
      if (!check_extent(*outb, {{p.limit, 1}}, 4, "the output", err)) return false;
    }
    prefetch_exposed(d);
    for (int r = 0; r < repeats; ++r) {
      std::string e = launch_rowwise(p, ctx);
      if (!e.empty()) { err = cuda_error(e); return false; }
    }
    k.last_path = 1;
    return true;
  }

  if (desc.id == KernelId::Matmul || desc.id == KernelId::SaeEncode) {
    GemmProblem p{};
    p.elt = desc.elt;
    int64_t M = get_int(d, Role::M, 0), N = get_int(d, Role::N, 0), K = get_int(d, Role::K, 0);
    const bool sae = desc.id == KernelId::SaeEncode;   // relu(x @ w + bias), row-major, no strides
    p.sam = get_int(d, Role::StrideAm, K);   // absent strides: row-major with unit inner stride
    p.sak = get_int(d, Role::StrideAk, 1);
    p.sbk = get_int(d, Role::StrideBk, N);
    p.sbn = get_int(d, Role::StrideBn, 1);
    p.scm = get_int(d, Role::StrideCm, N);
    p.scn = get_int(d, Role::StrideCn, 1);
    if (!nonneg(M, "M") || !nonneg(N, "N") || !nonneg(K, "K") || !nonneg(p.sam, "stride_am") ||
        !nonneg(p.sak, "stride_ak") || !nonneg(p.sbk, "stride_bk") || !nonneg(p.sbn, "stride_bn") ||
        !nonneg(p.scm, "stride_cm") || !nonneg(p.scn, "stride_cn"))
      return false;
    // Programs beyond the grid were never dispatched: their tiles stay untouched.
    if (desc.block_m > 0) M = std::min<int64_t>(M, gx * (int64_t)desc.block_m);
    if (desc.block_n > 0) N = std::min<int64_t>(N, gy * (int64_t)desc.block_n);
    p.M = M; p.N = N; p.K = K;
    BufferObj *A = buf(Role::A), *B = buf(Role::B), *C = buf(Role::C);
    if (!A || !B || !C || (sae && !buf(Role::BiasVec))) {
      err = invalid_argument(std::string(kernel_entry_name(desc.id)) + " was loaded from a descriptor without its buffer arguments");
      return false;
    }
    p.a = A->ptr; p.b = B->ptr; p.c = C->ptr;
    if (M == 0 || N == 0) return true;
    if (!check_int32(M, "M", err) || !check_int32(N, "N", err) || !check_int32(K, "K", err)) return false;
    if (!check_extent(*A, {{M, p.sam}, {K, p.sak}}, eb, "A", err)) return false;
    if (!check_extent(*B, {{K, p.sbk}, {N, p.sbn}}, eb, "B", err)) return false;
    if (!check_extent(*C, {{M, p.scm}, {N, p.scn}}, eb, "C", err)) return false;
    if (sae) {
      BufferObj* bias = buf(Role::BiasVec);
      if (!check_extent(*bias, {{N, 1}}, 4, "the bias", err)) return false;
      p.bias = (const float*)bias->ptr;
      p.relu = 1;
    }
    prefetch_exposed(d);
    std::string why;
    const bool f32 = p.elt == Elt::F32;
    bool tc = k.path_option != 1 && (f32 ? gemm_tf32_eligible(p, &why) : gemm_tc_eligible(p, &why));
    if (k.path_option == 2 && !tc) {
      err = invalid_argument("the tcgen05 path was required but this launch is not eligible: " + why);
      return false;
    }
    for (int r = 0; r < repeats; ++r) {
      std::string e = !tc ? launch_gemm_simt(p, ctx) : (f32 ? launch_gemm_tf32(p, ctx) : launch_gemm_tc(p, ctx));
      if (!e.empty()) { err = cuda_error(e); return false; }
    }
    k.last_path = tc ? 2 : 1;
    return true;
  }

  // ---- attention kernels ----
  AttnProblem p{};
  p.elt = desc.elt;
  p.sm_scale = d.sm_scale;
  p.stride_head = get_int(d, Role::StrideHead, 0);
  p.stride_seq = get_int(d, Role::StrideSeq, 0);
  p.stride_lse = get_int(d, Role::StrideLse, 0);
  p.n_ctx = get_int(d, Role::NCtx, 0);
  p.bh = gy;
  p.causal = desc.causal;
  p.head_dim = desc.head_dim > 0 ? desc.head_dim : (int)p.stride_seq;
  if (!nonneg(p.stride_head, "stride_head") || !nonneg(p.stride_seq, "stride_seq") ||
      !nonneg(p.stride_lse, "stride_lse") || !nonneg(p.n_ctx, "n_ctx"))
    return false;
  if (p.head_dim <= 0 || p.head_dim > 256) {
    err = invalid_argument("head dimension " + std::to_string(p.head_dim) +
                           " is outside the supported range 1...256");
    return false;
  }
  int block_rows = desc.id == KernelId::AttnBwdDkdv ? desc.block_n : desc.block_m;
  p.rows = p.n_ctx;
  if (block_rows > 0) p.rows = std::min<int64_t>(p.n_ctx, gx * (int64_t)block_rows);
  if (p.n_ctx == 0 || p.rows == 0) return true;
  if (!check_int32(p.n_ctx, "n_ctx", err) || !check_int32(p.bh, "grid_y (batch*heads)", err)) return false;
  auto data = [&](Role r, const char* what, const void** slot) {
    BufferObj* b = buf(r);
    if (!b) return true;
    if (!check_extent(*b, {{p.bh, p.stride_head}, {p.n_ctx, p.stride_seq}, {p.head_dim, 1}}, eb, what, err)) return false;
    *slot = b->ptr;
    return true;
  };
  auto stat = [&](Role r, const char* what, const void** slot) {
    BufferObj* b = buf(r);
    if (!b) return true;
    if (!check_extent(*b, {{p.bh, p.stride_lse}, {p.n_ctx, 1}}, 4, what, err)) return false;
    *slot = b->ptr;
    return true;
  };
  const void *dq = nullptr, *dk = nullptr, *dv = nullptr, *lse = nullptr, *delta = nullptr;
  if (!data(Role::Q, "Q", &p.q) || !data(Role::Kt, "K", &p.k) || !data(Role::V, "V", &p.v) ||
      !data(Role::O, "O", &p.o) || !data(Role::DO, "dO", &p.d_o) || !data(Role::DQ, "dQ", &dq) ||
      !data(Role::DK, "dK", &dk) || !data(Role::DV, "dV", &dv) || !stat(Role::L, "L", &lse) ||
      !stat(Role::Delta, "Delta", &delta))
    return false;
  p.lse = (float*)lse;
  p.delta = (const float*)delta;
  prefetch_exposed(d);
  std::string why, e;
  bool tc = false, f32 = false;     // fused 16-bit tcgen05 kernel / fp32 contractions as 3xTF32 GEMMs
  for (int r = 0; r < repeats; ++r) {
    switch (desc.id) {
      case KernelId::AttnFwd:
        p.out0 = (void*)p.o;
        tc = k.path_option != 1 && attn_fwd_tc_eligible(p, &why);
        f32 = !tc && k.path_option != 1 && attn_f32_tc_eligible(p, k.path_option == 2, &why);
        if (k.path_option == 2 && !tc && !f32) goto not_eligible;
        e = tc ? launch_attn_fwd_tc(p, ctx) : (f32 ? launch_attn_fwd_f32_tc(p, ctx) : launch_attn_fwd_simt(p, ctx));
        break;
      case KernelId::AttnBwdPreprocess:
        p.out0 = (void*)delta;
        tc = false;
        e = launch_attn_bwd_preprocess(p, ctx);
        break;
      case KernelId::AttnBwdDq:
        p.out0 = (void*)dq;
        tc = k.path_option != 1 && attn_bwd_tc_eligible(p, &why);
        f32 = !tc && k.path_option != 1 && attn_f32_tc_eligible(p, k.path_option == 2, &why);
        if (k.path_option == 2 && !tc && !f32) goto not_eligible;
        e = tc ? launch_attn_bwd_dq_tc(p, ctx) : (f32 ? launch_attn_bwd_dq_f32_tc(p, ctx) : launch_attn_bwd_dq_simt(p, ctx));
        break;
      case KernelId::AttnBwdDkdv:
        p.out0 = (void*)dk;
        p.out1 = (void*)dv;
        tc = k.path_option != 1 && attn_bwd_tc_eligible(p, &why);
        f32 = !tc && k.path_option != 1 && attn_f32_tc_eligible(p, k.path_option == 2, &why);
        if (k.path_option == 2 && !tc && !f32) goto not_eligible;
        e = tc ? launch_attn_bwd_dkdv_tc(p, ctx)
               : (f32 ? launch_attn_bwd_dkdv_f32_tc(p, ctx) : launch_attn_bwd_dkdv_simt(p, ctx));
        break;
      default:
        e = "unknown kernel";
    }
    if (!e.empty()) { err = cuda_error(e); return false; }
  }
  k.last_path = (tc || f32) ? 2 : 1;
  note.armed = true;
  return true;
not_eligible:
  err = invalid_argument("the tcgen05 path was required but this launch is not eligible: " + why);
  return false;
}

int32_t do_launch(int64_t kernel, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
                  const int32_t* kinds, const int64_t* values, int32_t argc, int repeats, bool wait,
                  float* elapsed_ms) {
  std::string err;
  auto k = lookup_as<KernelObj>(kernel, ObjKind::Kernel, err);
  if (!k) { store_error(err); return -1; }
  if (elapsed_ms) {
    if (!bind_device(err)) { store_error(err); return -1; }
    cudaEventRecord(g_dev.ev_begin, g_dev.stream);
  }
  if (!enqueue(*k, gx, gy, gz, threads, kinds, values, argc, repeats, err)) {
    store_error(err);
    return -1;
  }
  if (elapsed_ms) cudaEventRecord(g_dev.ev_end, g_dev.stream);
  if (wait) {
    if (!bind_device(err) || !sync_stream(err)) { store_error(err); return -1; }
    if (elapsed_ms) cudaEventElapsedTime(elapsed_ms, g_dev.ev_begin, g_dev.ev_end);
  }
  return 0;
}

int32_t do_copy(int64_t buffer, int64_t offset, const void* host, int64_t length, bool to_device,
                bool wait, bool side_stream = false) {
  // NULL / negative bounds are refused before the handle is looked at
  // (Compiler.swift:354-357).
  if (!host || length < 0 || offset < 0) {
    store_error(invalid_argument("buffer copy received invalid bounds"));
    return -1;
  }
  std::string err;
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return -1; }
  if ((__int128)offset + (__int128)length > (__int128)b->length) {
    store_error(invalid_argument("copy of " + std::to_string(length) + " bytes at offset " +
                                 std::to_string(offset) + " exceeds the " +
                                 std::to_string(b->length) + "-byte buffer"));
    return -1;
  }
  if (length == 0) return 0;
  if (!bind_device(err)) { store_error(err); return -1; }
  char* dev = (char*)b->ptr + offset;
  std::unique_lock<std::recursive_mutex> guard(g_dev.order_lock);
  cudaStream_t copy_stream = g_dev.stream;
  if (side_stream && !to_device) {
    // after everything enqueued so far, but not in the way of what is enqueued next
    cudaEventRecord(g_dev.ev_read, g_dev.stream);
    cudaStreamWaitEvent(g_dev.read_stream, g_dev.ev_read, 0);
    copy_stream = g_dev.read_stream;
    g_dev.reads_in_flight = true;
    if (!b->read_async_since_write) g_dev.read_back.push_back(b);
    b->read_async_since_write = true;
  }
  if (side_stream && to_device) {
    // ahead of the kernels enqueued so far, except the last one that took this buffer
    g_dev.async_writes = true;
    copy_stream = g_dev.write_stream;
    if (b->last_launch) {
      const int slot = (int)(b->last_launch % Device::kEventRing);
      if (g_dev.launch_event_number[slot] == b->last_launch) {
        cudaStreamWaitEvent(g_dev.write_stream, g_dev.launch_events[slot], 0);
      } else {
        // launched before events were being recorded, or more than a ring ago: wait for
        // everything enqueued so far
        cudaEventRecord(g_dev.ev_order, g_dev.stream);
        cudaStreamWaitEvent(g_dev.write_stream, g_dev.ev_order, 0);
      }
    }
    if (b->read_async_since_write) {
      cudaEventRecord(g_dev.ev_order, g_dev.read_stream);
      cudaStreamWaitEvent(g_dev.write_stream, g_dev.ev_order, 0);
    }
  }
  cudaError_t e = to_device
      ? cudaMemcpyAsync(dev, host, (size_t)length, cudaMemcpyDefault, copy_stream)
      : cudaMemcpyAsync((void*)host, dev, (size_t)length, cudaMemcpyDefault, copy_stream);
  if (e != cudaSuccess) {
    store_error(cuda_error(std::string("buffer copy failed: ") + cudaGetErrorString(e)));
    return -1;
  }
  if (side_stream && to_device) {
    // everything enqueued on the library's stream from here on comes after the copy
    const int slot = (int)(++g_dev.write_number % Device::kEventRing);
    cudaEventRecord(g_dev.write_events[slot], g_dev.write_stream);
    cudaStreamWaitEvent(g_dev.stream, g_dev.write_events[slot], 0);
  }
  guard.unlock();
  if (wait && !sync_stream(err)) { store_error(err); return -1; }
  return 0;
}

}  // namespace

// ===========================================================================
// Exports
// ===========================================================================
extern "C" {

char* tm_version(void) { return dup_string("0.0.1"); }

void tm_free(void* ptr) { std::free(ptr); }

char* tm_last_error(void) {
  std::lock_guard<std::mutex> guard(g_error_lock);
  std::string out = g_has_error ? g_error : std::string("no error");
  g_error.clear();
  g_has_error = false;
  return dup_string(out);
}

int32_t tm_is_active(void) {
  std::string err;
  return ensure_device(err) ? 1 : 0;
}

int32_t tm_is_usable(void) { return unusable_reason().empty() ? 1 : 0; }

char* tm_unusable_reason(void) {
  const std::string& why = unusable_reason();
  return why.empty() ? nullptr : dup_string(why);
}

char* tm_device_name(void) {
  std::string err;
  if (!ensure_device(err)) return nullptr;
  return dup_string(g_dev.prop.name);
}

char* tm_emit_msl(const char* ttir, int32_t num_simdgroups) {
  if (!ttir) {
    store_error(invalid_argument("tm_emit_msl received a NULL module"));
    return nullptr;
  }
  std::vector<KernelDesc> kernels;
  std::string err;
  if (!scan_module(ttir, num_simdgroups, kernels, err)) {
    store_error(err);
    return nullptr;
  }
  return dup_string(descriptor_text(kernels));
}

char* tm_kernel_info(const char* ttir, int32_t num_simdgroups) {
  if (!ttir) {
    store_error(invalid_argument("tm_kernel_info received a NULL module"));
    return nullptr;
  }
  std::vector<KernelDesc> kernels;
  std::string err;
  if (!scan_module(ttir, num_simdgroups, kernels, err)) {
    store_error(err);
    return nullptr;
  }
  return dup_string(kernel_info_json(kernels));
}

int64_t tm_compile_msl(const char* source) {
  if (!source) {
    store_error(invalid_argument("tm_compile_msl received NULL source"));
    return 0;
  }
  auto lib = std::make_shared<LibraryObj>();
  std::string err;
  if (!parse_descriptor(source, lib->kernels, err)) {
    store_error(err);
    return 0;
  }
  return g_handles.insert(lib);
}

int64_t tm_load_metallib(const void* bytes, int64_t length) {
  if (!bytes || length <= 0) {
    store_error(invalid_argument("tm_load_metallib received an empty image"));
    return 0;
  }
  // A binary of this platform - a cubin (ELF) or a fatbin - is loaded as it is: the caller's own
  // kernels behind the same launch call, which is what a metallib is to the reference
  // (Compiler.swift:250-262).  Anything else must be the text tm_emit_msl produced.
  const unsigned char* head = (const unsigned char*)bytes;
  const bool elf = length >= 4 && head[0] == 0x7f && head[1] == 'E' && head[2] == 'L' && head[3] == 'F';
  const bool fatbin = length >= 4 && head[0] == 0x50 && head[1] == 0xed && head[2] == 0x55 && head[3] == 0xba;
  if (elf || fatbin) {
    std::string err;
    if (!bind_device(err)) { store_error(err); return 0; }
    auto lib = std::make_shared<LibraryObj>();
    lib->image_bytes.assign((const char*)bytes, (size_t)length);
    cudaError_t e = cudaLibraryLoadData(&lib->image, lib->image_bytes.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    // (modules load lazily: counting the entry points is what makes the driver read the image)
    unsigned int entries = 0;
    if (e == cudaSuccess) e = cudaLibraryGetKernelCount(&entries, lib->image);
    if (e != cudaSuccess || entries == 0) {
      cudaGetLastError();
      store_error(cuda_error(std::string("could not load metallib: ") +
                             (e != cudaSuccess ? cudaGetErrorString(e) : "the image holds no kernels")));
      return 0;
    }
    return g_handles.insert(lib);
  }
  std::string text((const char*)bytes, (size_t)length);
  auto lib = std::make_shared<LibraryObj>();
  std::string err;
  if (!parse_descriptor(text, lib->kernels, err)) {
    store_error(cuda_error("could not load metallib: the image is not a tmcuda kernel descriptor"));
    return 0;
  }
  return g_handles.insert(lib);
}

int32_t tm_release_library(int64_t library) { return g_handles.remove(library) ? 0 : -1; }

int64_t tm_load_kernel(int64_t library, const char* name) {
  if (!name) {
    store_error(invalid_argument("tm_load_kernel received a NULL kernel name"));
    return 0;
  }
  std::string err;
  auto lib = lookup_as<LibraryObj>(library, ObjKind::Library, err);
  if (!lib) { store_error(err); return 0; }
  if (lib->image) {
    if (!bind_device(err)) { store_error(err); return 0; }
    cudaKernel_t entry = nullptr;
    if (cudaLibraryGetKernel(&entry, lib->image, name) != cudaSuccess || !entry) {
      cudaGetLastError();
      std::vector<std::string> names;
      unsigned int count = 0;
      if (cudaLibraryGetKernelCount(&count, lib->image) == cudaSuccess && count) {
        std::vector<cudaKernel_t> all(count);
        if (cudaLibraryEnumerateKernels(all.data(), count, lib->image) == cudaSuccess) {
          for (cudaKernel_t one : all) {
            const char* n = nullptr;
            if (cudaFuncGetName(&n, (const void*)one) == cudaSuccess && n) names.push_back(n);
          }
        }
      }
      cudaGetLastError();
      std::sort(names.begin(), names.end());
      std::string available;
      for (auto& n : names) available += (available.empty() ? "" : ", ") + n;
      store_error(cuda_error(std::string("kernel '") + name + "' not found in library (available: " + available + ")"));
      return 0;
    }
    auto obj = std::make_shared<KernelObj>();
    obj->binary = entry;
    obj->binary_name = name;
    obj->owner = lib;
    cudaFuncAttributes attr{};
    if (cudaFuncGetAttributes(&attr, (const void*)entry) == cudaSuccess) obj->max_threads = attr.maxThreadsPerBlock;
    for (size_t i = 0;; ++i) {
      size_t offset = 0, size = 0;
      if (cudaFuncGetParamInfo((const void*)entry, i, &offset, &size) != cudaSuccess) break;
      obj->param_sizes.push_back(size);
    }
    cudaGetLastError();
    return g_handles.insert(obj);
  }
  for (auto& k : lib->kernels) {
    if (std::string(name) == kernel_entry_name(k.id)) {
      auto obj = std::make_shared<KernelObj>();
      obj->desc = k;
      // $TMCUDA_FORCE_PATH=simt|tcgen05 presets the "path" option of every kernel.
      if (const char* force = std::getenv("TMCUDA_FORCE_PATH")) {
        if (std::string(force) == "simt") obj->path_option = 1;
        else if (std::string(force) == "tcgen05") obj->path_option = 2;
      }
      return g_handles.insert(obj);
    }
  }
  std::vector<std::string> names;
  for (auto& k : lib->kernels) names.push_back(kernel_entry_name(k.id));
  std::sort(names.begin(), names.end());
  std::string available;
  for (auto& n : names) available += (available.empty() ? "" : ", ") + n;
  store_error(cuda_error(std::string("kernel '") + name + "' not found in library (available: " +
                         (available.empty() ? "none" : available) + ")"));
  return 0;
}

int64_t tm_kernel_max_threads(int64_t kernel) {
  std::string err;
  auto k = lookup_as<KernelObj>(kernel, ObjKind::Kernel, err);
  if (!k) { store_error(err); return -1; }
  return k->binary ? k->max_threads : 1024;
}

int32_t tm_release_kernel(int64_t kernel) { return g_handles.remove(kernel) ? 0 : -1; }

int64_t tm_alloc_buffer(int64_t nbytes) {
  if (nbytes <= 0) {
    store_error(invalid_argument("buffer length must be positive, got " + std::to_string(nbytes)));
    return 0;
  }
  std::string err;
  if (!bind_device(err)) { store_error(err); return 0; }
  auto b = std::make_shared<BufferObj>();
  cudaError_t e = cudaMallocManaged(&b->ptr, (size_t)nbytes, cudaMemAttachGlobal);
  if (e != cudaSuccess) {
    cudaGetLastError();
    b->ptr = nullptr;
    store_error(cuda_error("could not allocate a " + std::to_string(nbytes) + "-byte shared buffer: " +
                           cudaGetErrorString(e)));
    return 0;
  }
  b->length = nbytes;
  // Resident on the device, and zero-filled like a new MTLBuffer.
  cudaMemPrefetchAsync(b->ptr, (size_t)nbytes, g_dev.ordinal, g_dev.stream);
  cudaMemsetAsync(b->ptr, 0, (size_t)nbytes, g_dev.stream);
  e = cudaStreamSynchronize(g_dev.stream);
  if (e != cudaSuccess) {
    store_error(cuda_error(std::string("could not initialise the buffer: ") + cudaGetErrorString(e)));
    return 0;
  }
  return g_handles.insert(b);
}

void* tm_buffer_contents(int64_t buffer) {
  std::string err;
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return nullptr; }
  if (b->device_only) {
    store_error(invalid_argument("buffer " + std::to_string(buffer) +
                                 " is device-only memory and has no host-addressable contents"));
    return nullptr;
  }
  b->host_exposed = true;
  return b->ptr;
}

int64_t tm_buffer_length(int64_t buffer) {
  std::string err;
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return -1; }
  return b->length;
}

int32_t tm_buffer_write(int64_t buffer, int64_t offset, const void* source, int64_t length) {
  return do_copy(buffer, offset, source, length, true, true);
}

int32_t tm_buffer_read(int64_t buffer, int64_t offset, void* destination, int64_t length) {
  return do_copy(buffer, offset, destination, length, false, true);
}

int32_t tm_free_buffer(int64_t buffer) {
  std::string err;
  // The object is destroyed (cudaFree) with the library's device current.
  if (g_dev.ok) cudaSetDevice(g_dev.ordinal);
  return g_handles.remove(buffer) ? 0 : -1;
}

int32_t tm_launch(int64_t kernel, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
                  const int32_t* kinds, const int64_t* values, int32_t argc) {
  return do_launch(kernel, gx, gy, gz, threads, kinds, values, argc, 1, true, nullptr);
}

int64_t tm_live_handle_count(void) { return g_handles.count(); }

// ---- additive -------------------------------------------------------------

int32_t tmx_set_device(int32_t ordinal) {
  std::lock_guard<std::mutex> guard(g_dev.lock);
  if (g_dev.tried && g_dev.ordinal != ordinal) {
    store_error(invalid_argument("tmx_set_device must be called before the first use of the device"));
    return -1;
  }
  if (ordinal < 0) {
    store_error(invalid_argument("device ordinal must not be negative"));
    return -1;
  }
  g_dev.ordinal = ordinal;
  return 0;
}

int32_t tmx_get_device(void) {
  std::string err;
  if (!ensure_device(err)) { store_error(err); return -1; }
  return g_dev.ordinal;
}

int32_t tmx_sm_count(void) {
  std::string err;
  if (!ensure_device(err)) { store_error(err); return -1; }
  return g_dev.prop.multiProcessorCount;
}

int32_t tmx_kernel_set_option(int64_t kernel, const char* name, int64_t value) {
  std::string err;
  auto k = lookup_as<KernelObj>(kernel, ObjKind::Kernel, err);
  if (!k) { store_error(err); return -1; }
  if (!name) { store_error(invalid_argument("tmx_kernel_set_option received a NULL name")); return -1; }
  if (k->binary) {
    store_error(invalid_argument("kernels of a binary image take no options"));
    return -1;
  }
  std::string n(name);
  if (n == "causal") {
    if (k->desc.id == KernelId::Matmul || k->desc.id == KernelId::AttnBwdPreprocess || is_rowwise(k->desc.id)) {
      store_error(invalid_argument(std::string("option 'causal' does not apply to ") +
                                   kernel_entry_name(k->desc.id)));
      return -1;
    }
    k->desc.causal = value != 0;
    return 0;
  }
  if (n == "path") {
    if (value < 0 || value > 2) {
      store_error(invalid_argument("option 'path' takes 0, 1 or 2"));
      return -1;
    }
    k->path_option = (int)value;
    return 0;
  }
  store_error(invalid_argument("unknown kernel option '" + n + "'"));
  return -1;
}

int32_t tmx_kernel_last_path(int64_t kernel) {
  std::string err;
  auto k = lookup_as<KernelObj>(kernel, ObjKind::Kernel, err);
  if (!k) { store_error(err); return -1; }
  return k->last_path;
}

int32_t tmx_launch_async(int64_t kernel, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
                         const int32_t* kinds, const int64_t* values, int32_t argc) {
  return do_launch(kernel, gx, gy, gz, threads, kinds, values, argc, 1, false, nullptr);
}

int32_t tmx_launch_timed(int64_t kernel, int64_t gx, int64_t gy, int64_t gz, int64_t threads,
                         const int32_t* kinds, const int64_t* values, int32_t argc, int32_t repeats,
                         float* elapsed_ms) {
  if (!elapsed_ms || repeats <= 0) {
    store_error(invalid_argument("tmx_launch_timed needs repeats > 0 and a result pointer"));
    return -1;
  }
  return do_launch(kernel, gx, gy, gz, threads, kinds, values, argc, repeats, true, elapsed_ms);
}

int32_t tmx_synchronize(void) {
  std::string err;
  if (!bind_device(err) || !sync_stream(err)) { store_error(err); return -1; }
  return 0;
}

int32_t tmx_buffer_write_async(int64_t buffer, int64_t offset, const void* source, int64_t length) {
  return do_copy(buffer, offset, source, length, true, false, true);
}

int32_t tmx_buffer_read_async(int64_t buffer, int64_t offset, void* destination, int64_t length) {
  return do_copy(buffer, offset, destination, length, false, false, true);
}

int32_t tmx_buffer_fill(int64_t buffer, int64_t offset, int32_t byte, int64_t length) {
  std::string err;
  if (length < 0 || offset < 0) {
    store_error(invalid_argument("buffer fill received invalid bounds"));
    return -1;
  }
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return -1; }
  if ((__int128)offset + (__int128)length > (__int128)b->length) {
    store_error(invalid_argument("fill of " + std::to_string(length) + " bytes at offset " +
                                 std::to_string(offset) + " exceeds the " +
                                 std::to_string(b->length) + "-byte buffer"));
    return -1;
  }
  if (!bind_device(err)) { store_error(err); return -1; }
  cudaError_t e = cudaMemsetAsync((char*)b->ptr + offset, byte, (size_t)length, g_dev.stream);
  if (e != cudaSuccess) {
    store_error(cuda_error(std::string("buffer fill failed: ") + cudaGetErrorString(e)));
    return -1;
  }
  return 0;
}

int32_t tmx_timer_begin(void) {
  std::string err;
  if (!bind_device(err)) { store_error(err); return -1; }
  cudaEventRecord(g_dev.ev_begin, g_dev.stream);
  // uploads enqueued from here on belong to the timed region: they start behind its first event
  cudaStreamWaitEvent(g_dev.write_stream, g_dev.ev_begin, 0);
  return 0;
}

int32_t tmx_timer_end(float* elapsed_ms) {
  std::string err;
  if (!elapsed_ms) { store_error(invalid_argument("tmx_timer_end needs a result pointer")); return -1; }
  if (!bind_device(err)) { store_error(err); return -1; }
  join_reads();
  cudaEventRecord(g_dev.ev_end, g_dev.stream);
  if (!sync_stream(err)) { store_error(err); return -1; }
  cudaEventElapsedTime(elapsed_ms, g_dev.ev_begin, g_dev.ev_end);
  return 0;
}

int64_t tmx_launch_count(void) { return g_dev.launches; }

// Plain device memory (cudaMalloc), for buffers that are handed to other device-side
// libraries (NCCL wants ordinary device allocations) and never read through a host pointer.
int64_t tmx_alloc_device_buffer(int64_t nbytes) {
  if (nbytes <= 0) {
    store_error(invalid_argument("buffer length must be positive, got " + std::to_string(nbytes)));
    return 0;
  }
  std::string err;
  if (!bind_device(err)) { store_error(err); return 0; }
  auto b = std::make_shared<BufferObj>();
  cudaError_t e = cudaMalloc(&b->ptr, (size_t)nbytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    b->ptr = nullptr;
    store_error(cuda_error("could not allocate a " + std::to_string(nbytes) + "-byte device buffer: " +
                           cudaGetErrorString(e)));
    return 0;
  }
  b->length = nbytes;
  b->device_only = true;
  cudaMemsetAsync(b->ptr, 0, (size_t)nbytes, g_dev.stream);
  cudaStreamSynchronize(g_dev.stream);
  return g_handles.insert(b);
}

// The library's CUDA stream (a cudaStream_t), so that other stream-ordered work (an NCCL
// collective, a torch op) can be enqueued in order with the launches instead of behind a
// host synchronisation.
void* tmx_stream_handle(void) {
  std::string err;
  if (!bind_device(err)) { store_error(err); return nullptr; }
  return (void*)g_dev.stream;
}

// The device address of a buffer (for interop with libraries that take raw pointers).
void* tmx_buffer_device_pointer(int64_t buffer) {
  std::string err;
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return nullptr; }
  return b->ptr;
}

// fp32 C = A @ B with no device allocation anywhere on the path: the scratch for the
// 3xTF32 operand split is a fixed array inside the library.  Same arithmetic as
// matmul_kernel launched through tm_launch on fp32 buffers.
int32_t tmx_matmul_f32_static(int64_t a, int64_t b, int64_t c, int64_t M, int64_t N, int64_t K,
                              int64_t stride_am, int64_t stride_ak, int64_t stride_bk,
                              int64_t stride_bn, int64_t stride_cm, int64_t stride_cn) {
  std::string err;
  auto A = lookup_as<BufferObj>(a, ObjKind::Buffer, err);
  auto B = A ? lookup_as<BufferObj>(b, ObjKind::Buffer, err) : nullptr;
  auto C = B ? lookup_as<BufferObj>(c, ObjKind::Buffer, err) : nullptr;
  if (!C) { store_error(err); return -1; }
  if (M <= 0 || N <= 0 || K <= 0 || stride_am < 0 || stride_ak < 0 || stride_bk < 0 || stride_bn < 0 ||
      stride_cm < 0 || stride_cn < 0) {
    store_error(invalid_argument("tmx_matmul_f32_static needs positive extents and non-negative strides"));
    return -1;
  }
  GemmProblem p{};
  p.elt = Elt::F32;
  p.a = A->ptr; p.b = B->ptr; p.c = C->ptr;
  p.M = M; p.N = N; p.K = K;
  p.sam = stride_am; p.sak = stride_ak; p.sbk = stride_bk; p.sbn = stride_bn;
  p.scm = stride_cm; p.scn = stride_cn;
  if (!check_int32(M, "M", err) || !check_int32(N, "N", err) || !check_int32(K, "K", err) ||
      !check_extent(*A, {{M, p.sam}, {K, p.sak}}, 4, "A", err) ||
      !check_extent(*B, {{K, p.sbk}, {N, p.sbn}}, 4, "B", err) ||
      !check_extent(*C, {{M, p.scm}, {N, p.scn}}, 4, "C", err)) {
    store_error(err);
    return -1;
  }
  std::string why;
  if (M < 128 || N < 64 || K < 32) {
    store_error(invalid_argument("tmx_matmul_f32_static takes problems of at least 128 x 64 x 32"));
    return -1;
  }
  if (!bind_device(err)) { store_error(err); return -1; }
  if (g_dev.prop.major != 10) {
    store_error(cuda_error("this device is not sm_100; libtmcuda holds sm_100a code only"));
    return -1;
  }
  Decoded d;
  d.buffers[(int)Role::A] = A;
  d.buffers[(int)Role::B] = B;
  d.buffers[(int)Role::C] = C;
  prefetch_exposed(d);
  std::string e = run_gemm_tf32_static(p, launch_ctx(), g_dev.ordinal);
  if (!e.empty()) {
    store_error(e.rfind("the operand split needs", 0) == 0 ? invalid_argument(e) : cuda_error(e));
    return -1;
  }
  note_launch(std::vector<BufferObj*>{A.get(), B.get(), C.get()});
  if (!sync_stream(err)) { store_error(err); return -1; }
  return 0;
}

int64_t tmx_matmul_f32_static_capacity(void) { return (int64_t)gemm_tf32_static_capacity(); }

// The once-per-device set-up of tmx_matmul_f32_static on its own: resolves the fixed array's
// device address, which under lazy module loading is also when the driver reserves the array
// and the kernel images on the GPU.  A host calls this before it hands the rest of device
// memory to its own pool; afterwards tmx_matmul_f32_static changes the amount of free device
// memory by nothing.
int32_t tmx_matmul_f32_static_prepare(void) {
  std::string err;
  if (!bind_device(err)) { store_error(err); return -1; }
  std::string e = prepare_gemm_tf32_static(g_dev.ordinal);
  if (!e.empty()) { store_error(cuda_error(e)); return -1; }
  return 0;
}

// Free and total bytes of device memory as the driver reports them (cudaMemGetInfo).
int32_t tmx_device_memory(int64_t* free_bytes, int64_t* total_bytes) {
  std::string err;
  if (!free_bytes || !total_bytes) {
    store_error(invalid_argument("tmx_device_memory needs two result pointers"));
    return -1;
  }
  if (!bind_device(err)) { store_error(err); return -1; }
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  if (e != cudaSuccess) {
    store_error(cuda_error(std::string("cudaMemGetInfo: ") + cudaGetErrorString(e)));
    return -1;
  }
  *free_bytes = (int64_t)f;
  *total_bytes = (int64_t)t;
  return 0;
}

// ---- buffers shared between the processes of a multi-GPU job --------------------------

// The 64-byte token another process on this machine turns into a mapping of this buffer
// (cudaIpcGetMemHandle).  Only plain device memory (tmx_alloc_device_buffer) can be shared.
int32_t tmx_ipc_export(int64_t buffer, void* handle64) {
  std::string err;
  if (!handle64) { store_error(invalid_argument("tmx_ipc_export needs 64 bytes for the handle")); return -1; }
  auto b = lookup_as<BufferObj>(buffer, ObjKind::Buffer, err);
  if (!b) { store_error(err); return -1; }
  if (!b->device_only || b->imported) {
    store_error(invalid_argument("only a buffer made by tmx_alloc_device_buffer can be exported"));
    return -1;
  }
  if (!bind_device(err)) { store_error(err); return -1; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, b->ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    store_error(cuda_error(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e)));
    return -1;
  }
  std::memcpy(handle64, &h, 64);
  return 0;
}

// Maps another process's exported buffer (of `nbytes` bytes) into this one and enables peer
// access to its GPU.  The result is a device-only buffer handle: kernels may write it, copies
// may read it; tm_free_buffer unmaps it.
int64_t tmx_ipc_import(const void* handle64, int64_t nbytes) {
  std::string err;
  if (!handle64 || nbytes <= 0) {
    store_error(invalid_argument("tmx_ipc_import needs a handle and a positive length"));
    return 0;
  }
  if (!bind_device(err)) { store_error(err); return 0; }
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  auto b = std::make_shared<BufferObj>();
  cudaError_t e = cudaIpcOpenMemHandle(&b->ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    b->ptr = nullptr;
    store_error(cuda_error(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e)));
    return 0;
  }
  b->length = nbytes;
  b->device_only = true;
  b->imported = true;
  return g_handles.insert(b);
}

int64_t tmx_gather_flag_bytes(void) { return (int64_t)kGatherFlagSlots * kGatherMaxRanks * 4; }

// Row-sharded matmul whose epilogue replicates C (see include/tm.h).  Enqueues and returns.
int32_t tmx_matmul_gathered(int64_t kernel, int64_t a, int64_t b, const int64_t* c_replicas,
                            const int64_t* flag_buffers, int32_t world, int32_t rank, int64_t row0,
                            int64_t rows, int64_t N, int64_t K, int32_t slot, uint32_t epoch,
                            int32_t wait_for_peers) {
  std::string err;
  auto fail = [&](const std::string& m) { store_error(m); return -1; };
  auto k = lookup_as<KernelObj>(kernel, ObjKind::Kernel, err);
  if (!k) return fail(err);
  if (k->binary || k->desc.id != KernelId::Matmul || k->desc.elt == Elt::F32)
    return fail(invalid_argument("tmx_matmul_gathered takes a 16-bit matmul_kernel"));
  if (!c_replicas || !flag_buffers || world < 1 || world > kGatherMaxRanks || rank < 0 || rank >= world)
    return fail(invalid_argument("tmx_matmul_gathered needs 1...8 ranks, this rank among them, and their buffers"));
  if (slot < 0 || slot >= kGatherFlagSlots || epoch == 0)
    return fail(invalid_argument("flag slot must be 0...63 and the epoch positive"));
  if (row0 < 0 || rows <= 0 || N <= 0 || K <= 0)
    return fail(invalid_argument("tmx_matmul_gathered needs positive extents"));
  auto A = lookup_as<BufferObj>(a, ObjKind::Buffer, err);
  auto B = A ? lookup_as<BufferObj>(b, ObjKind::Buffer, err) : nullptr;
  if (!B) return fail(err);
  GemmGather g{};
  std::vector<std::shared_ptr<BufferObj>> keep;
  for (int r = 0; r < world; ++r) {
    auto c = lookup_as<BufferObj>(c_replicas[r], ObjKind::Buffer, err);
    auto f = c ? lookup_as<BufferObj>(flag_buffers[r], ObjKind::Buffer, err) : nullptr;
    if (!f) return fail(err);
    if (!c->device_only || !f->device_only)
      return fail(invalid_argument("copies of C and flag arrays must be plain device memory"));
    if (!check_int32(row0 + rows, "row0 + rows", err) || !check_int32(N, "N", err) || !check_int32(K, "K", err) ||
        !check_extent(*c, {{row0 + rows, N}, {N, 1}}, 2, "a copy of C", err))
      return fail(err);
    if (f->length < tmx_gather_flag_bytes())
      return fail(invalid_argument("a flag array is smaller than tmx_gather_flag_bytes()"));
    g.replica[r] = c->ptr;
    g.flags[r] = (uint32_t*)f->ptr;
    keep.push_back(c);
    keep.push_back(f);
  }
  if (!check_extent(*A, {{rows, K}, {K, 1}}, 2, "A", err) || !check_extent(*B, {{K, N}, {N, 1}}, 2, "B", err))
    return fail(err);
  if (!bind_device(err)) return fail(err);
  {
    const std::string& why = unusable_reason();
    if (!why.empty()) return fail(cuda_error(why));
  }
  if (!g_dev.gather_counter) {
    cudaError_t e = cudaMalloc((void**)&g_dev.gather_counter, sizeof(unsigned int));
    if (e != cudaSuccess) { cudaGetLastError(); return fail(cuda_error(std::string("cudaMalloc: ") + cudaGetErrorString(e))); }
    cudaMemsetAsync(g_dev.gather_counter, 0, sizeof(unsigned int), g_dev.stream);
  }
  GemmProblem p{};
  p.elt = k->desc.elt;
  p.a = A->ptr;
  p.b = B->ptr;
  p.c = (char*)g.replica[rank] + (size_t)row0 * (size_t)N * 2;
  p.M = rows; p.N = N; p.K = K;
  p.sam = K; p.sak = 1; p.sbk = N; p.sbn = 1; p.scm = N; p.scn = 1;
  std::string why;
  if (!gemm_tc_eligible(p, &why))
    return fail(invalid_argument("this problem cannot take the tcgen05 kernel: " + why));
  g.finished = g_dev.gather_counter;
  g.world = world; g.rank = rank; g.slot = slot; g.epoch = epoch;
  g.wait_for_peers = wait_for_peers;
  g.wait_budget_cycles = 0;
  if (const char* env = std::getenv("TMCUDA_GATHER_WAIT_CYCLES")) g.wait_budget_cycles = std::atoll(env);
  // finished tiles leave through TMA stores; $TMCUDA_GATHER_TMA_STORE=0 selects plain st.global
  g.tma_store = 1;
  if (const char* env = std::getenv("TMCUDA_GATHER_TMA_STORE")) g.tma_store = std::atoi(env) != 0;
  std::string e = launch_gemm_tc_gathered(p, g, launch_ctx());
  if (!e.empty()) return fail(cuda_error(e));
  k->last_path = 2;
  std::vector<BufferObj*> launch_buffers{A.get(), B.get()};
  for (auto& kept : keep) launch_buffers.push_back(kept.get());
  note_launch(launch_buffers);
  return 0;
}

// ---- failure-path aids ------------------------------------------------------

// Runs the bounded-wait self-test kernel (csrc/selftest.cu) with the given cycle budget and
// waits for it.  The kernel's waits run out and it records that in the device status word;
// the word is left in place, so the next tm_launch / tmx_synchronize / copy reports it.
int32_t tmx_selftest_bounded_wait(int64_t budget_cycles, int32_t* results) {
  std::string err;
  if (!results || budget_cycles <= 0 || budget_cycles > 2000000000ll) {
    store_error(invalid_argument("tmx_selftest_bounded_wait needs a result pointer and a budget of 1...2e9 cycles"));
    return -1;
  }
  if (!bind_device(err)) { store_error(err); return -1; }
  {
    const std::string& why = unusable_reason();
    if (!why.empty()) { store_error(cuda_error(why)); return -1; }
  }
  int got[2] = {0, 0};
  std::string e = launch_bounded_wait_selftest(launch_ctx(), (long long)budget_cycles, got);
  if (!e.empty()) { store_error(cuda_error("self-test launch failed: " + e)); return -1; }
  results[0] = got[0];
  results[1] = got[1];
  return 0;
}

// The work lists the persistent attention kernels would walk for a problem shape, for
// inspection: kind 0 forward (256-row query blocks), 1 dq, 2 dkdv (128-row tiles).  Writes up
// to `capacity` (batch-head, block) pairs into items_out, ctas + 1 offsets into begin_out and
// the modelled cost of each CTA into load_out (any of them may be NULL); returns the number of
// items, or -1.  Needs no device.
int64_t tmx_debug_attention_schedule(int32_t kind, int32_t bh, int32_t rows, int32_t n_ctx, int32_t causal,
                                     int32_t ctas, int32_t* items_out, int64_t capacity, int32_t* begin_out,
                                     int64_t* load_out) {
  if (kind < 0 || kind > 2 || bh <= 0 || rows <= 0 || n_ctx <= 0 || ctas <= 0) {
    store_error(invalid_argument("tmx_debug_attention_schedule needs kind 0...2 and positive extents"));
    return -1;
  }
  const AttnWorkList list = kind == 0 ? schedule_attn_fwd(bh, rows, n_ctx, causal != 0, ctas)
                                      : schedule_attn_bwd(bh, rows, n_ctx, causal != 0, kind == 1, ctas);
  const int64_t n = (int64_t)list.items.size();
  if (items_out) {
    for (int64_t i = 0; i < n && i < capacity; ++i) {
      items_out[2 * i] = list.items[i].bh;
      items_out[2 * i + 1] = list.items[i].block;
    }
  }
  if (begin_out) std::copy(list.begin.begin(), list.begin.end(), begin_out);
  if (load_out) std::copy(list.load.begin(), list.load.end(), load_out);
  return n;
}

// Writes a device status record from the host, as if a kernel's bounded wait had given up.
int32_t tmx_debug_inject_status(int32_t code, int32_t where, int32_t block, int32_t extra) {
  std::string err;
  if (!bind_device(err)) { store_error(err); return -1; }
  g_dev.status->where = (unsigned)where;
  g_dev.status->block = (unsigned)block;
  g_dev.status->extra = (unsigned)extra;
  g_dev.status->code = (unsigned)code;
  return 0;
}

}  // extern "C"
