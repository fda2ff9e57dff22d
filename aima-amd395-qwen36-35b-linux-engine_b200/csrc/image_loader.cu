// Striped weight image: layout planner, builder and scatter ingest of tensors (or per-rank expert
// slabs of tensors) from two lane files into device memory, with the reference's XOR / SUM
// checksum over 64-bit words evaluated on the device.
//
// Follows the reference's image tooling:
//   layout    "deterministic LPT by descending aligned bytes then tensor name; assign to the
//             lower-total lane with lane0 winning ties", extents aligned to 4096 bytes
//             (engine/production-striped-image-manifest.json: layout.algorithm, entries[*])
//   builder   benchmarks/shape-lab/native/src/striped_image_builder.cpp:97-135 (plan geometry),
//             :137-147 (checksum over uint64 words)
//   ingest    torch_owned_striped_tensor_scatter_ingest, the C ABI of
//             benchmarks/shape-lab/native/src/torch_owned_striped_image_loader.hip.cpp:127-135:
//             per lane one reader with two pinned buffers and two streams, chunked reads,
//             asynchronous copies to caller-owned device tensors, device checksum (:95-123)
// Differences that expert parallelism needs: a tensor entry may name any 4096-aligned byte range
// of an extent (rank r of W loads experts [r*256/W, (r+1)*256/W) of an expert tensor, which is one
// contiguous range because the expert index is the outermost dimension), and the expected
// checksum is optional.
#include "../../include/aima_moe.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace aima {
void set_last_error_message(const char* message);
}

namespace {

constexpr uint64_t kImageAlignment = 4096;
constexpr int kLanes = 2;
constexpr int kBuffersPerLane = 2;
constexpr int kChecksumThreads = 256;

int image_fail(int status, const std::string& message) {
  aima::set_last_error_message(message.c_str());
  return status;
}

// XOR and wrapping SUM are order-free: every range is cut into pieces of at most kChecksumPieceWords
// words, one block per piece, 16-byte loads, four in flight per thread; block results join by atomics.
struct ChecksumTask {
  const uint64_t* data;     // 16-byte aligned
  uint64_t words;
};
constexpr uint64_t kChecksumPieceWords = (2u << 20) / 8;

__global__ void __launch_bounds__(kChecksumThreads)
image_checksum_kernel(const ChecksumTask* __restrict__ tasks,
                      unsigned long long* __restrict__ xor_out, unsigned long long* __restrict__ sum_out) {
  __shared__ unsigned long long xor_values[kChecksumThreads];
  __shared__ unsigned long long sum_values[kChecksumThreads];
  const ChecksumTask task = tasks[blockIdx.x];
  const ulonglong2* pairs = reinterpret_cast<const ulonglong2*>(task.data);
  const uint64_t n_pairs = task.words / 2;
  unsigned long long x0 = 0, x1 = 0, s0 = 0, s1 = 0;
  uint64_t index = threadIdx.x;
  for (; index + 3 * kChecksumThreads < n_pairs; index += 4 * kChecksumThreads) {
    const ulonglong2 a = __ldcs(pairs + index);
    const ulonglong2 b = __ldcs(pairs + index + kChecksumThreads);
    const ulonglong2 c = __ldcs(pairs + index + 2 * kChecksumThreads);
    const ulonglong2 d = __ldcs(pairs + index + 3 * kChecksumThreads);
    x0 ^= a.x ^ b.x ^ c.x ^ d.x;
    x1 ^= a.y ^ b.y ^ c.y ^ d.y;
    s0 += a.x + b.x + c.x + d.x;
    s1 += a.y + b.y + c.y + d.y;
  }
  for (; index < n_pairs; index += kChecksumThreads) {
    const ulonglong2 a = __ldcs(pairs + index);
    x0 ^= a.x; x1 ^= a.y; s0 += a.x; s1 += a.y;
  }
  if ((task.words & 1u) != 0 && threadIdx.x == 0) {
    const unsigned long long last = task.data[task.words - 1];
    x0 ^= last;
    s0 += last;
  }
  xor_values[threadIdx.x] = x0 ^ x1;
  sum_values[threadIdx.x] = s0 + s1;
  __syncthreads();
  for (int offset = kChecksumThreads / 2; offset > 0; offset >>= 1) {
    if (threadIdx.x < offset) {
      xor_values[threadIdx.x] ^= xor_values[threadIdx.x + offset];
      sum_values[threadIdx.x] += sum_values[threadIdx.x + offset];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    atomicXor(xor_out, xor_values[0]);
    atomicAdd(sum_out, sum_values[0]);
  }
}

struct LaneJob {
  uint64_t lane_offset;     // where the range starts in the lane file
  uint64_t bytes;
  uint8_t* destination;     // device
};

struct LaneReader {
  std::string path;
  std::vector<LaneJob> jobs;
  uint64_t chunk_bytes = 0;
  int device = 0;
  std::string error;
  uint64_t bytes_read = 0;
  bool direct = false;

  void run() {
    void* buffers[kBuffersPerLane] = {};
    cudaStream_t streams[kBuffersPerLane] = {};
    cudaEvent_t copied[kBuffersPerLane] = {};
    int descriptor = -1;
    auto fail = [&](const std::string& what) { if (error.empty()) error = what; };
    do {
      if (cudaSetDevice(device) != cudaSuccess) { fail("cudaSetDevice in a lane reader"); break; }
      // direct I/O when the file system allows it: every range is 4096-aligned in offset, the pinned
      // buffers are page-aligned; the tail of a range is read up to the next 4096 boundary
      descriptor = open(path.c_str(), O_RDONLY | O_DIRECT);
      direct = descriptor >= 0;
      if (descriptor < 0) descriptor = open(path.c_str(), O_RDONLY);
      if (descriptor < 0) { fail("cannot open " + path); break; }
      bool ok = true;
      for (int b = 0; b < kBuffersPerLane && ok; ++b) {
        ok = cudaHostAlloc(&buffers[b], chunk_bytes, cudaHostAllocDefault) == cudaSuccess &&
             cudaStreamCreateWithFlags(&streams[b], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&copied[b], cudaEventDisableTiming) == cudaSuccess;
      }
      if (!ok) { fail("pinned buffers / streams of a lane reader"); break; }
      int turn = 0;
      bool used[kBuffersPerLane] = {};
      for (const LaneJob& job : jobs) {
        uint64_t done = 0;
        while (done < job.bytes && error.empty()) {
          const uint64_t want = std::min<uint64_t>(chunk_bytes, job.bytes - done);
          const uint64_t padded = (want + kImageAlignment - 1) / kImageAlignment * kImageAlignment;
          const int b = turn;
          turn = (turn + 1) % kBuffersPerLane;
          if (used[b] && cudaEventSynchronize(copied[b]) != cudaSuccess) { fail("cudaEventSynchronize"); break; }
          uint64_t got = 0;
          while (got < want) {
            const ssize_t n = pread(descriptor, static_cast<uint8_t*>(buffers[b]) + got,
                                    static_cast<size_t>((direct ? padded : want) - got),
                                    static_cast<off_t>(job.lane_offset + done + got));
            if (n < 0 && direct && errno == EINVAL && got == 0) {
              // the file system accepted O_DIRECT at open but not for this read: go on buffered
              close(descriptor);
              descriptor = open(path.c_str(), O_RDONLY);
              direct = false;
              if (descriptor < 0) break;
              continue;
            }
            if (n <= 0) break;
            got += static_cast<uint64_t>(n);
          }
          if (got < want) { fail("short read from " + path); break; }
          if (cudaMemcpyAsync(job.destination + done, buffers[b], want, cudaMemcpyHostToDevice, streams[b]) != cudaSuccess ||
              cudaEventRecord(copied[b], streams[b]) != cudaSuccess) { fail("cudaMemcpyAsync from a lane buffer"); break; }
          used[b] = true;
          done += want;
          bytes_read += want;
        }
        if (!error.empty()) break;
      }
    } while (false);
    for (int b = 0; b < kBuffersPerLane; ++b) {
      if (streams[b] != nullptr) { cudaStreamSynchronize(streams[b]); cudaStreamDestroy(streams[b]); }
      if (copied[b] != nullptr) cudaEventDestroy(copied[b]);
      if (buffers[b] != nullptr) cudaFreeHost(buffers[b]);
    }
    if (descriptor >= 0) close(descriptor);
  }
};

}  // namespace

extern "C" {

#define AIMA_EXPORT __attribute__((visibility("default")))

AIMA_EXPORT int aima_moe_image_plan(const uint64_t* payload_bytes, const char* const* names, uint64_t count,
                                    uint32_t* lane, uint64_t* lane_offset, uint64_t* aggregate_offset,
                                    uint64_t* lane_bytes) {
  if (payload_bytes == nullptr || names == nullptr || lane == nullptr || lane_offset == nullptr ||
      aggregate_offset == nullptr || lane_bytes == nullptr || count == 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image plan: null argument or no tensors");
  std::vector<uint64_t> order(count);
  std::vector<uint64_t> aligned(count);
  for (uint64_t i = 0; i < count; ++i) {
    if (payload_bytes[i] == 0 || names[i] == nullptr)
      return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image plan: empty tensor or null name");
    order[i] = i;
    aligned[i] = (payload_bytes[i] + kImageAlignment - 1) / kImageAlignment * kImageAlignment;
  }
  std::sort(order.begin(), order.end(), [&](uint64_t a, uint64_t b) {
    if (aligned[a] != aligned[b]) return aligned[a] > aligned[b];
    return std::strcmp(names[a], names[b]) < 0;
  });
  uint64_t totals[kLanes] = {0, 0};
  for (uint64_t i : order) {
    const int l = totals[0] <= totals[1] ? 0 : 1;
    lane[i] = static_cast<uint32_t>(l);
    lane_offset[i] = totals[l];
    totals[l] += aligned[i];
  }
  for (uint64_t i = 0; i < count; ++i) aggregate_offset[i] = (lane[i] == 0 ? 0 : totals[0]) + lane_offset[i];
  lane_bytes[0] = totals[0];
  lane_bytes[1] = totals[1];
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_image_checksum_host(const void* data, uint64_t bytes, uint64_t* xor_value,
                                             uint64_t* sum_value) {
  if (data == nullptr || xor_value == nullptr || sum_value == nullptr || bytes % 8 != 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image checksum: null argument or bytes not a multiple of 8");
  const uint64_t* words = static_cast<const uint64_t*>(data);
  uint64_t x = *xor_value, s = *sum_value;
  for (uint64_t i = 0; i < bytes / 8; ++i) { x ^= words[i]; s += words[i]; }
  *xor_value = x;
  *sum_value = s;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_image_build(const char* lane0_path, const char* lane1_path,
                                     const void* const* host_tensors, const uint64_t* payload_bytes,
                                     const uint32_t* lane, const uint64_t* lane_offset, uint64_t count,
                                     const uint64_t* lane_bytes, uint64_t* xor_value, uint64_t* sum_value) {
  if (lane0_path == nullptr || lane1_path == nullptr || host_tensors == nullptr || payload_bytes == nullptr ||
      lane == nullptr || lane_offset == nullptr || lane_bytes == nullptr || count == 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image build: null argument");
  const char* paths[kLanes] = {lane0_path, lane1_path};
  int descriptors[kLanes] = {-1, -1};
  uint64_t x = 0, s = 0;
  int status = AIMA_MOE_OK;
  for (int l = 0; l < kLanes && status == AIMA_MOE_OK; ++l) {
    descriptors[l] = open(paths[l], O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (descriptors[l] < 0 || ftruncate(descriptors[l], static_cast<off_t>(lane_bytes[l])) != 0)
      status = image_fail(AIMA_MOE_ERR_INTERNAL, std::string("image build: cannot create ") + paths[l]);
  }
  for (uint64_t i = 0; i < count && status == AIMA_MOE_OK; ++i) {
    if (lane[i] >= kLanes || lane_offset[i] % kImageAlignment != 0 || payload_bytes[i] % 8 != 0 ||
        lane_offset[i] + payload_bytes[i] > lane_bytes[lane[i]]) {
      status = image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image build: extent outside its lane or misaligned");
      break;
    }
    uint64_t done = 0;
    while (done < payload_bytes[i]) {
      const ssize_t n = pwrite(descriptors[lane[i]], static_cast<const uint8_t*>(host_tensors[i]) + done,
                               static_cast<size_t>(std::min<uint64_t>(payload_bytes[i] - done, 1u << 30)),
                               static_cast<off_t>(lane_offset[i] + done));
      if (n <= 0) { status = image_fail(AIMA_MOE_ERR_INTERNAL, "image build: short write"); break; }
      done += static_cast<uint64_t>(n);
    }
    if (status == AIMA_MOE_OK) aima_moe_image_checksum_host(host_tensors[i], payload_bytes[i], &x, &s);
  }
  for (int l = 0; l < kLanes; ++l) {
    if (descriptors[l] >= 0) { fsync(descriptors[l]); close(descriptors[l]); }
  }
  if (status == AIMA_MOE_OK) {
    if (xor_value != nullptr) *xor_value = x;
    if (sum_value != nullptr) *sum_value = s;
  }
  return status;
}

AIMA_EXPORT int aima_moe_image_scatter_ingest(const char* lane0_path, const char* lane1_path,
                                              const uint64_t* aggregate_offsets, const uint64_t* payload_bytes,
                                              const uint64_t* destination_ptrs, uint64_t tensor_count,
                                              uint64_t lane0_bytes, uint64_t lane1_bytes, uint64_t chunk_bytes,
                                              int check_expected, uint64_t expected_xor, uint64_t expected_sum,
                                              aima_moe_image_ingest_result* result) {
  if (lane0_path == nullptr || lane1_path == nullptr || aggregate_offsets == nullptr || payload_bytes == nullptr ||
      destination_ptrs == nullptr || result == nullptr || tensor_count == 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image ingest: null argument");
  if (lane0_bytes == 0 || lane1_bytes == 0 || lane0_bytes % kImageAlignment != 0 || lane1_bytes % kImageAlignment != 0 ||
      chunk_bytes == 0 || chunk_bytes % kImageAlignment != 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image ingest: lane sizes and chunk size must be multiples of 4096");
  std::memset(result, 0, sizeof *result);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    return image_fail(AIMA_MOE_ERR_NO_DEVICE, "image ingest: no CUDA device (there is no CPU fallback)");
  }
  LaneReader readers[kLanes];
  readers[0].path = lane0_path;
  readers[1].path = lane1_path;
  uint64_t total = 0;
  std::vector<ChecksumTask> tasks;
  for (uint64_t i = 0; i < tensor_count; ++i) {
    const uint64_t offset = aggregate_offsets[i], bytes = payload_bytes[i];
    if (destination_ptrs[i] == 0 || offset % kImageAlignment != 0 || bytes == 0 || bytes % 8 != 0 ||
        destination_ptrs[i] % 16 != 0)
      return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image ingest: range " + std::to_string(i) +
                        " is empty, misaligned or has no destination");
    const int l = offset < lane0_bytes ? 0 : 1;
    const uint64_t in_lane = offset - (l == 0 ? 0 : lane0_bytes);
    if (in_lane + bytes > (l == 0 ? lane0_bytes : lane1_bytes))
      return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image ingest: range " + std::to_string(i) + " crosses the end of its lane");
    cudaPointerAttributes attributes{};
    if (cudaPointerGetAttributes(&attributes, reinterpret_cast<const void*>(destination_ptrs[i])) != cudaSuccess ||
        (attributes.type != cudaMemoryTypeDevice && attributes.type != cudaMemoryTypeManaged)) {
      (void)cudaGetLastError();
      return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image ingest: destination " + std::to_string(i) + " is not device memory");
    }
    readers[l].jobs.push_back({in_lane, bytes, reinterpret_cast<uint8_t*>(destination_ptrs[i])});
    for (uint64_t word = 0; word < bytes / 8; word += kChecksumPieceWords)
      tasks.push_back({reinterpret_cast<const uint64_t*>(destination_ptrs[i]) + word,
                       std::min<uint64_t>(kChecksumPieceWords, bytes / 8 - word)});
    total += bytes;
  }
  for (LaneReader& reader : readers) { reader.chunk_bytes = chunk_bytes; reader.device = device; }
  const auto started = std::chrono::steady_clock::now();
  std::thread second([&] { readers[1].run(); });
  readers[0].run();
  second.join();
  const double read_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - started).count();
  for (const LaneReader& reader : readers)
    if (!reader.error.empty()) return image_fail(AIMA_MOE_ERR_INTERNAL, "image ingest: " + reader.error);

  // device checksum over everything that was written
  ChecksumTask* device_tasks = nullptr;
  unsigned long long* device_words = nullptr;
  cudaError_t error = cudaMalloc(&device_tasks, sizeof(ChecksumTask) * tasks.size());
  if (error == cudaSuccess) error = cudaMalloc(&device_words, 16);
  if (error == cudaSuccess) error = cudaMemset(device_words, 0, 16);
  if (error == cudaSuccess)
    error = cudaMemcpy(device_tasks, tasks.data(), sizeof(ChecksumTask) * tasks.size(), cudaMemcpyHostToDevice);
  cudaEvent_t begin = nullptr, end = nullptr;
  float checksum_ms = 0.0f;
  if (error == cudaSuccess) error = cudaEventCreate(&begin);
  if (error == cudaSuccess) error = cudaEventCreate(&end);
  if (error == cudaSuccess) {
    cudaEventRecord(begin, nullptr);
    image_checksum_kernel<<<static_cast<unsigned>(tasks.size()), kChecksumThreads>>>(device_tasks, device_words,
                                                                                   device_words + 1);
    cudaEventRecord(end, nullptr);
    error = cudaGetLastError();
    if (error == cudaSuccess) error = cudaEventSynchronize(end);
    if (error == cudaSuccess) cudaEventElapsedTime(&checksum_ms, begin, end);
  }
  unsigned long long words[2] = {0, 0};
  if (error == cudaSuccess) error = cudaMemcpy(words, device_words, 16, cudaMemcpyDeviceToHost);
  if (begin != nullptr) cudaEventDestroy(begin);
  if (end != nullptr) cudaEventDestroy(end);
  cudaFree(device_tasks);
  cudaFree(device_words);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return image_fail(static_cast<int>(error), std::string("image ingest: device checksum: ") + cudaGetErrorString(error));
  }
  result->bytes = total;
  result->read_ms = read_ms;
  result->checksum_ms = checksum_ms;
  result->xor_value = words[0];
  result->sum_value = words[1];
  result->direct_io = (readers[0].direct ? 1u : 0u) | (readers[1].direct ? 2u : 0u);
  if (check_expected && (words[0] != expected_xor || words[1] != expected_sum))
    return image_fail(AIMA_MOE_ERR_INTERNAL, "image ingest: checksum of the loaded bytes differs from the expected one");
  return AIMA_MOE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Safetensors shards as the source of an image: header index and a builder that copies extents
// from source files.  Format: 8-byte little-endian header length N, N bytes of JSON
// {"tensor": {"dtype": "BF16", "shape": [..], "data_offsets": [begin, end]}, ..., "__metadata__": {..}},
// then the data section; data_offsets are relative to its start.  The reference's manifest records
// the same two numbers per tensor (source_data_offset_bytes = 8 + N, source_offset_bytes =
// source_data_offset_bytes + begin; engine/production-striped-image-manifest.json entries[*]) and its
// builder copies [source offset, + payload) to the planned extent
// (benchmarks/shape-lab/native/src/striped_image_builder.cpp:97-135, 149-200).
// ---------------------------------------------------------------------------
namespace {

struct JsonCursor {
  const char* p;
  const char* end;
  bool ok = true;
  void skip_ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p; }
  bool eat(char c) { skip_ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool peek(char c) { skip_ws(); return p < end && *p == c; }
  std::string string() {
    std::string out;
    skip_ws();
    if (p >= end || *p != '"') { ok = false; return out; }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': out.push_back('?'); p += (p + 4 < end) ? 4 : 0; break;   // names are ASCII in practice
          default: out.push_back(*p); break;
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  uint64_t number() {
    skip_ws();
    uint64_t value = 0;
    bool any = false;
    while (p < end && *p >= '0' && *p <= '9') { value = value * 10 + static_cast<uint64_t>(*p - '0'); ++p; any = true; }
    if (!any) ok = false;
    return value;
  }
  void skip_value() {   // any JSON value
    skip_ws();
    if (p >= end) { ok = false; return; }
    if (*p == '"') { (void)string(); return; }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = (*p == '{') ? '}' : ']';
      ++p;
      if (eat(close)) return;
      do {
        if (open == '{') { (void)string(); if (!eat(':')) { ok = false; return; } }
        skip_value();
        if (!ok) return;
      } while (eat(','));
      if (!eat(close)) ok = false;
      return;
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;   // number, true, false, null
  }
};

}  // namespace

extern "C" {

AIMA_EXPORT int aima_moe_safetensors_index(const char* path, aima_moe_safetensors_entry* entries,
                                           uint64_t capacity, uint64_t* count) {
  if (path == nullptr || count == nullptr || (entries == nullptr && capacity != 0))
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "safetensors index: null argument");
  *count = 0;
  const int descriptor = open(path, O_RDONLY);
  if (descriptor < 0) return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, std::string("safetensors index: cannot open ") + path);
  uint64_t header_bytes = 0;
  const off_t file_bytes = lseek(descriptor, 0, SEEK_END);
  if (pread(descriptor, &header_bytes, 8, 0) != 8 || header_bytes == 0 || header_bytes > (1ull << 30) ||
      static_cast<uint64_t>(file_bytes) < 8 + header_bytes) {
    close(descriptor);
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, std::string("safetensors index: bad header length in ") + path);
  }
  std::string header(header_bytes, '\0');
  uint64_t got = 0;
  while (got < header_bytes) {
    const ssize_t n = pread(descriptor, &header[got], header_bytes - got, static_cast<off_t>(8 + got));
    if (n <= 0) break;
    got += static_cast<uint64_t>(n);
  }
  close(descriptor);
  if (got < header_bytes) return image_fail(AIMA_MOE_ERR_INTERNAL, "safetensors index: short read of the header");
  const uint64_t data_start = 8 + header_bytes;
  JsonCursor json{header.data(), header.data() + header.size()};
  if (!json.eat('{')) return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "safetensors index: header is not a JSON object");
  uint64_t found = 0;
  if (!json.peek('}')) {
    do {
      const std::string name = json.string();
      if (!json.ok || !json.eat(':')) { json.ok = false; break; }
      if (name == "__metadata__") { json.skip_value(); continue; }
      aima_moe_safetensors_entry entry{};
      bool have_offsets = false;
      if (!json.eat('{')) { json.ok = false; break; }
      do {
        const std::string key = json.string();
        if (!json.ok || !json.eat(':')) { json.ok = false; break; }
        if (key == "dtype") {
          const std::string dtype = json.string();
          std::snprintf(entry.dtype, sizeof entry.dtype, "%s", dtype.c_str());
        } else if (key == "shape") {
          if (!json.eat('[')) { json.ok = false; break; }
          if (!json.peek(']')) {
            do {
              const uint64_t extent = json.number();
              if (entry.rank < 4) entry.shape[entry.rank] = extent;
              ++entry.rank;
            } while (json.ok && json.eat(','));
          }
          if (!json.eat(']')) json.ok = false;
        } else if (key == "data_offsets") {
          if (!json.eat('[')) { json.ok = false; break; }
          entry.data_begin = data_start + json.number();
          if (!json.eat(',')) json.ok = false;
          entry.data_end = data_start + json.number();
          if (!json.eat(']')) json.ok = false;
          have_offsets = true;
        } else {
          json.skip_value();
        }
      } while (json.ok && json.eat(','));
      if (!json.ok || !json.eat('}')) { json.ok = false; break; }
      if (!have_offsets || entry.rank > 4 || entry.data_end < entry.data_begin ||
          entry.data_end > static_cast<uint64_t>(file_bytes) || name.size() >= sizeof entry.name)
        return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "safetensors index: tensor " + name + " has a bad entry");
      std::snprintf(entry.name, sizeof entry.name, "%s", name.c_str());
      if (found < capacity) entries[found] = entry;
      ++found;
    } while (json.ok && json.eat(','));
  }
  if (!json.ok || !json.eat('}'))
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, std::string("safetensors index: malformed header in ") + path);
  *count = found;
  if (found > capacity && capacity != 0)
    return image_fail(AIMA_MOE_ERR_CAPACITY, "safetensors index: more tensors than the entry array holds");
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_image_build_from_files(const char* lane0_path, const char* lane1_path,
                                                const char* const* source_paths, const uint64_t* source_offsets,
                                                const uint64_t* payload_bytes, const uint32_t* lane,
                                                const uint64_t* lane_offset, uint64_t count,
                                                const uint64_t* lane_bytes, uint64_t* xor_value, uint64_t* sum_value) {
  if (lane0_path == nullptr || lane1_path == nullptr || source_paths == nullptr || source_offsets == nullptr ||
      payload_bytes == nullptr || lane == nullptr || lane_offset == nullptr || lane_bytes == nullptr || count == 0)
    return image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image build: null argument");
  const char* paths[kLanes] = {lane0_path, lane1_path};
  int descriptors[kLanes] = {-1, -1};
  int status = AIMA_MOE_OK;
  for (int l = 0; l < kLanes && status == AIMA_MOE_OK; ++l) {
    descriptors[l] = open(paths[l], O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (descriptors[l] < 0 || ftruncate(descriptors[l], static_cast<off_t>(lane_bytes[l])) != 0)
      status = image_fail(AIMA_MOE_ERR_INTERNAL, std::string("image build: cannot create ") + paths[l]);
  }
  std::vector<uint8_t> buffer(16u << 20);
  uint64_t x = 0, s = 0;
  for (uint64_t i = 0; i < count && status == AIMA_MOE_OK; ++i) {
    if (source_paths[i] == nullptr || lane[i] >= kLanes || lane_offset[i] % kImageAlignment != 0 ||
        payload_bytes[i] == 0 || payload_bytes[i] % 8 != 0 || lane_offset[i] + payload_bytes[i] > lane_bytes[lane[i]]) {
      status = image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "image build: extent " + std::to_string(i) + " is misaligned or outside its lane");
      break;
    }
    const int source = open(source_paths[i], O_RDONLY);
    if (source < 0) { status = image_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, std::string("image build: cannot open ") + source_paths[i]); break; }
    uint64_t done = 0;
    while (done < payload_bytes[i] && status == AIMA_MOE_OK) {
      const uint64_t want = std::min<uint64_t>(buffer.size(), payload_bytes[i] - done);
      uint64_t got = 0;
      while (got < want) {
        const ssize_t n = pread(source, buffer.data() + got, want - got, static_cast<off_t>(source_offsets[i] + done + got));
        if (n <= 0) break;
        got += static_cast<uint64_t>(n);
      }
      if (got < want) { status = image_fail(AIMA_MOE_ERR_INTERNAL, std::string("image build: short read from ") + source_paths[i]); break; }
      uint64_t put = 0;
      while (put < want) {
        const ssize_t n = pwrite(descriptors[lane[i]], buffer.data() + put, want - put, static_cast<off_t>(lane_offset[i] + done + put));
        if (n <= 0) break;
        put += static_cast<uint64_t>(n);
      }
      if (put < want) { status = image_fail(AIMA_MOE_ERR_INTERNAL, "image build: short write"); break; }
      aima_moe_image_checksum_host(buffer.data(), want, &x, &s);
      done += want;
    }
    close(source);
  }
  for (int l = 0; l < kLanes; ++l) {
    if (descriptors[l] >= 0) { fsync(descriptors[l]); close(descriptors[l]); }
  }
  if (status == AIMA_MOE_OK) {
    if (xor_value != nullptr) *xor_value = x;
    if (sum_value != nullptr) *sum_value = s;
  }
  return status;
}

}  // extern "C"
