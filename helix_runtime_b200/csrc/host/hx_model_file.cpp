// Reader for Helix's native model file ("HELIXLM1"), host code only.
//
// The container (src/model/format.cpp:40-52, 526-550 of the reference project) is
// little-endian and fully canonical: a 128-byte header that carries the model's sizes, a
// directory of 80-byte entries, then the float32 payloads, each starting on a 64-byte
// boundary with zero bytes between them.  Everything in the header and the directory except
// the checksums follows from the model's sizes, so this reader works from a PLAN: it reads the
// sizes, lays out the file a writer would have produced for them, and compares the file's
// fields with that plan one by one, each mismatch with its own message.  Checksums are
// FNV-1a (64-bit) over the header with its checksum field zeroed plus the directory, and over
// each payload's bytes (src/model/format.cpp:341-355, 586-590).
//
// Interface: open maps the file and checks header and directory; verify walks the padding
// and the payloads (zero padding, checksum, finite values) on several threads; the tensors
// are then read in place from the mapping.  Nothing here needs a GPU.
#include "hx_model_file.h"

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

thread_local std::string g_error;

int fail(int code, const char* format, ...) {
  char buffer[512];
  va_list arguments;
  va_start(arguments, format);
  vsnprintf(buffer, sizeof buffer, format, arguments);
  va_end(arguments);
  g_error = buffer;
  return code;
}

constexpr unsigned char kMagic[8] = {'H', 'E', 'L', 'I', 'X', 'L', 'M', '1'};
constexpr uint64_t kHeaderBytes = 128;
constexpr uint64_t kEntryBytes = 80;
constexpr uint64_t kAlignment = 64;
constexpr uint64_t kFnvOffset = 14695981039346656037ull;
constexpr uint64_t kFnvPrime = 1099511628211ull;
constexpr uint32_t kGlobalLayer = 0xffffffffu;
constexpr uint64_t kChecksumField = kHeaderBytes - 8;

uint64_t fnv1a(const unsigned char* bytes, size_t count, uint64_t hash) {
  for (size_t i = 0; i < count; ++i) {
    hash ^= bytes[i];
    hash *= kFnvPrime;
  }
  return hash;
}

uint64_t little(const unsigned char* at, int width) {
  uint64_t value = 0;
  for (int i = width - 1; i >= 0; --i) value = (value << 8) | at[i];
  return value;
}

uint64_t round_up(uint64_t value, uint64_t step) { return (value + step - 1) / step * step; }

// A fixed field of the header: where it is, how wide, what it must hold, and what to say.
struct FixedField {
  uint64_t offset;
  int width;
  uint64_t expected;
  const char* complaint;
};

constexpr FixedField kFixedFields[] = {
    {8, 4, 1, "unsupported format version"},
    {12, 4, 0x01020304u, "the endianness marker is not little-endian 0x01020304"},
    {16, 4, kHeaderBytes, "the header size field is not 128"},
    {20, 4, HX_MODEL_KIND_LLAMA, "the model kind is not one this reader knows"},
    {32, 8, kHeaderBytes, "the directory does not start behind the header"},
    {48, 8, kEntryBytes, "the directory entry size field is not 80"},
};

struct PlannedTensor {
  int role;
  uint32_t layer;
  int rank;
  uint64_t dims[4];
  uint64_t offset;
  uint64_t bytes;
};

const char* role_name(int role) {
  static const char* names[] = {"?", "token_embedding", "attention_norm", "query", "key", "value",
                                "attention_output", "ffn_norm", "gate", "up", "down", "final_norm",
                                "lm_head"};
  return role >= 1 && role <= 12 ? names[role] : names[0];
}

// The file a writer produces for these sizes: which tensors, in which order, where.
// Sizes are at most 2^32 each (checked by the caller), so a tensor's byte count fits 128 bits;
// `fits` turns false when one would not fit a file.
std::vector<PlannedTensor> plan_for(const hx_model_config& c, uint64_t* data_offset,
                                    uint64_t* file_bytes, bool* fits) {
  std::vector<PlannedTensor> plan;
  const uint64_t V = c.vocab_size, H = c.hidden_size, I = c.intermediate_size;
  *fits = true;
  auto add = [&plan, fits](int role, uint32_t layer, uint64_t rows, uint64_t columns) {
    const unsigned __int128 wide = static_cast<unsigned __int128>(rows) * (columns ? columns : 1) * 4;
    if (wide > (static_cast<unsigned __int128>(1) << 56)) *fits = false;
    PlannedTensor t{};
    t.role = role;
    t.layer = layer;
    t.rank = columns ? 2 : 1;
    t.dims[0] = rows;
    t.dims[1] = columns;
    t.bytes = rows * (columns ? columns : 1) * 4;
    plan.push_back(t);
  };
  add(HX_ROLE_TOKEN_EMBEDDING, kGlobalLayer, V, H);
  for (uint64_t layer = 0; layer < c.num_layers; ++layer) {
    const uint32_t l = static_cast<uint32_t>(layer);
    add(HX_ROLE_ATTENTION_NORM, l, H, 0);
    add(HX_ROLE_QUERY, l, H, H);
    add(HX_ROLE_KEY, l, H, H);
    add(HX_ROLE_VALUE, l, H, H);
    add(HX_ROLE_ATTENTION_OUTPUT, l, H, H);
    add(HX_ROLE_FFN_NORM, l, H, 0);
    add(HX_ROLE_GATE, l, H, I);
    add(HX_ROLE_UP, l, H, I);
    add(HX_ROLE_DOWN, l, I, H);
  }
  add(HX_ROLE_FINAL_NORM, kGlobalLayer, H, 0);
  add(HX_ROLE_LM_HEAD, kGlobalLayer, H, V);
  uint64_t cursor = round_up(kHeaderBytes + kEntryBytes * plan.size(), kAlignment);
  *data_offset = cursor;
  for (PlannedTensor& t : plan) {
    cursor = round_up(cursor, kAlignment);
    t.offset = cursor;
    cursor += t.bytes;
  }
  *file_bytes = cursor;
  return plan;
}

}  // namespace

struct hx_model_file {
  int descriptor = -1;
  const unsigned char* base = nullptr;
  uint64_t bytes = 0;
  hx_model_config config{};
  uint64_t data_offset = 0;
  std::vector<PlannedTensor> tensors;
  std::vector<uint64_t> checksums;
};

extern "C" {

const char* hx_host_last_error(void) { return g_error.c_str(); }

uint64_t hx_fnv1a64(const void* bytes, uint64_t count, uint64_t seed) {
  return fnv1a(static_cast<const unsigned char*>(bytes), count, seed ? seed : kFnvOffset);
}

void hx_model_file_close(hx_model_file* file) {
  if (file == nullptr) return;
  if (file->base != nullptr) munmap(const_cast<unsigned char*>(file->base), file->bytes);
  if (file->descriptor >= 0) close(file->descriptor);
  delete file;
}

int hx_model_file_open(const char* path, hx_model_file** out) {
  *out = nullptr;
  hx_model_file* file = new hx_model_file();
  struct Closer {
    hx_model_file* file;
    ~Closer() { hx_model_file_close(file); }
  } closer{file};

  file->descriptor = open(path, O_RDONLY | O_CLOEXEC);
  if (file->descriptor < 0)
    return fail(HX_FILE_IO, "could not open '%s' for reading: %s", path, strerror(errno));
  struct stat info {};
  if (fstat(file->descriptor, &info) != 0 || !S_ISREG(info.st_mode))
    return fail(HX_FILE_IO, "'%s' is not a regular file", path);
  file->bytes = static_cast<uint64_t>(info.st_size);
  if (file->bytes < kHeaderBytes)
    return fail(HX_FILE_FORMAT, "%s: the file is smaller than the 128-byte header", path);
  void* mapping = mmap(nullptr, file->bytes, PROT_READ, MAP_PRIVATE, file->descriptor, 0);
  if (mapping == MAP_FAILED)
    return fail(HX_FILE_IO, "could not map '%s': %s", path, strerror(errno));
  file->base = static_cast<const unsigned char*>(mapping);
  const unsigned char* header = file->base;

  if (memcmp(header, kMagic, sizeof kMagic) != 0)
    return fail(HX_FILE_FORMAT, "%s: the magic bytes are not HELIXLM1", path);
  for (const FixedField& field : kFixedFields) {
    const uint64_t found = little(header + field.offset, field.width);
    if (found != field.expected)
      return fail(HX_FILE_FORMAT, "%s: %s (found %llu)", path, field.complaint,
                  static_cast<unsigned long long>(found));
  }
  const uint64_t declared_bytes = little(header + 24, 8);
  if (declared_bytes != file->bytes)
    return fail(HX_FILE_FORMAT, "%s: the header declares %llu bytes, the file has %llu", path,
                static_cast<unsigned long long>(declared_bytes),
                static_cast<unsigned long long>(file->bytes));

  hx_model_config& c = file->config;
  c.model_kind = static_cast<uint32_t>(little(header + 20, 4));
  uint64_t* sizes[] = {&c.vocab_size, &c.hidden_size, &c.intermediate_size,
                       &c.num_layers, &c.num_heads,   &c.max_positions};
  const char* size_names[] = {"vocabulary size", "hidden size", "intermediate size",
                              "layer count", "attention head count", "maximum sequence length"};
  for (int i = 0; i < 6; ++i) {
    *sizes[i] = little(header + 64 + 8 * i, 8);
    // every size also bounds a product below: keep them where 64-bit arithmetic is exact
    if (*sizes[i] == 0 || *sizes[i] > (1ull << 32))
      return fail(HX_FILE_FORMAT, "%s: the %s in the header is %llu", path, size_names[i],
                  static_cast<unsigned long long>(*sizes[i]));
  }
  const uint32_t eps_bits = static_cast<uint32_t>(little(header + 112, 4));
  const uint32_t theta_bits = static_cast<uint32_t>(little(header + 116, 4));
  memcpy(&c.rms_norm_eps, &eps_bits, 4);
  memcpy(&c.rope_theta, &theta_bits, 4);
  if (!std::isfinite(c.rms_norm_eps) || !(c.rms_norm_eps > 0.0f) ||
      !std::isfinite(c.rope_theta) || !(c.rope_theta > 0.0f))
    return fail(HX_FILE_FORMAT, "%s: epsilon and rotary base must be positive and finite", path);
  if (c.hidden_size % c.num_heads != 0 || (c.hidden_size / c.num_heads) % 2 != 0)
    return fail(HX_FILE_FORMAT, "%s: hidden size %llu does not split into %llu even heads", path,
                static_cast<unsigned long long>(c.hidden_size),
                static_cast<unsigned long long>(c.num_heads));

  uint64_t planned_bytes = 0;
  if (c.num_layers > (1u << 20))
    return fail(HX_FILE_FORMAT, "%s: the layer count in the header is %llu", path,
                static_cast<unsigned long long>(c.num_layers));
  bool fits = true;
  file->tensors = plan_for(c, &file->data_offset, &planned_bytes, &fits);
  if (!fits) return fail(HX_FILE_FORMAT, "%s: the header's sizes describe an impossible file", path);
  const uint64_t count = little(header + 40, 8);
  if (count != file->tensors.size())
    return fail(HX_FILE_FORMAT, "%s: %llu tensors in the directory, a model of %llu layers has %zu",
                path, static_cast<unsigned long long>(count),
                static_cast<unsigned long long>(c.num_layers), file->tensors.size());
  if (kHeaderBytes + kEntryBytes * count > file->bytes)
    return fail(HX_FILE_FORMAT, "%s: the tensor directory runs past the end of the file", path);
  if (little(header + 56, 8) != file->data_offset)
    return fail(HX_FILE_FORMAT, "%s: the data offset is %llu, canonical is %llu", path,
                static_cast<unsigned long long>(little(header + 56, 8)),
                static_cast<unsigned long long>(file->data_offset));

  // metadata checksum: header with its checksum field as zeros, then the directory
  const unsigned char zeros[8] = {};
  uint64_t hash = fnv1a(header, kChecksumField, kFnvOffset);
  hash = fnv1a(zeros, 8, hash);
  hash = fnv1a(header + kHeaderBytes, kEntryBytes * count, hash);
  if (hash != little(header + kChecksumField, 8))
    return fail(HX_FILE_FORMAT, "%s: metadata checksum mismatch (header or directory damaged)",
                path);

  file->checksums.resize(count);
  for (uint64_t index = 0; index < count; ++index) {
    const unsigned char* entry = header + kHeaderBytes + kEntryBytes * index;
    const PlannedTensor& t = file->tensors[index];
    const char* name = role_name(t.role);
    if (little(entry, 4) != static_cast<uint64_t>(t.role) || little(entry + 4, 4) != t.layer)
      return fail(HX_FILE_FORMAT, "%s: directory entry %llu should be %s of layer %d", path,
                  static_cast<unsigned long long>(index), name, static_cast<int>(t.layer));
    if (little(entry + 8, 4) != 1)
      return fail(HX_FILE_FORMAT, "%s: %s has a dtype code other than float32", path, name);
    if (little(entry + 12, 4) != static_cast<uint64_t>(t.rank))
      return fail(HX_FILE_FORMAT, "%s: %s has rank %llu, expected %d", path, name,
                  static_cast<unsigned long long>(little(entry + 12, 4)), t.rank);
    for (int d = 0; d < 4; ++d)
      if (little(entry + 16 + 8 * d, 8) != t.dims[d])
        return fail(HX_FILE_FORMAT, "%s: %s has an unexpected shape", path, name);
    if (little(entry + 56, 8) != t.bytes)
      return fail(HX_FILE_FORMAT, "%s: %s has an invalid byte length", path, name);
    if (little(entry + 48, 8) != t.offset || little(entry + 64, 8) != kAlignment)
      return fail(HX_FILE_FORMAT, "%s: %s has a non-canonical payload offset or alignment", path,
                  name);
    file->checksums[index] = little(entry + 72, 8);
  }
  if (planned_bytes < file->bytes)
    return fail(HX_FILE_FORMAT, "%s: %llu trailing bytes behind the last payload", path,
                static_cast<unsigned long long>(file->bytes - planned_bytes));
  if (planned_bytes > file->bytes)
    return fail(HX_FILE_FORMAT, "%s: the payloads need %llu bytes, the file has %llu", path,
                static_cast<unsigned long long>(planned_bytes),
                static_cast<unsigned long long>(file->bytes));
  closer.file = nullptr;
  *out = file;
  return HX_FILE_OK;
}

int hx_model_file_config(const hx_model_file* file, hx_model_config* out) {
  *out = file->config;
  return HX_FILE_OK;
}

long long hx_model_file_tensor_count(const hx_model_file* file) {
  return static_cast<long long>(file->tensors.size());
}

int hx_model_file_tensor(const hx_model_file* file, long long index, hx_model_tensor* out) {
  if (index < 0 || static_cast<size_t>(index) >= file->tensors.size())
    return fail(HX_FILE_ARGUMENT, "tensor index %lld is outside the directory", index);
  const PlannedTensor& t = file->tensors[static_cast<size_t>(index)];
  out->role = t.role;
  out->layer = t.layer == kGlobalLayer ? -1 : static_cast<int>(t.layer);
  out->rank = t.rank;
  for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
  out->offset = t.offset;
  out->bytes = t.bytes;
  out->checksum = file->checksums[static_cast<size_t>(index)];
  out->data = file->base + t.offset;
  return HX_FILE_OK;
}

// Padding is zero, every payload hashes to its checksum and holds finite values only.
int hx_model_file_verify(const hx_model_file* file, int threads) {
  const size_t count = file->tensors.size();
  uint64_t cursor = kHeaderBytes + kEntryBytes * count;
  for (size_t index = 0; index < count; ++index) {
    const PlannedTensor& t = file->tensors[index];
    for (uint64_t at = cursor; at < t.offset; ++at)
      if (file->base[at] != 0)
        return fail(HX_FILE_FORMAT, "alignment padding before %s holds a non-zero byte",
                    role_name(t.role));
    cursor = t.offset + t.bytes;
  }
  std::atomic<size_t> next{0};
  std::atomic<int> bad_kind{0};       // 1 checksum, 2 non-finite
  std::atomic<size_t> bad_index{0};
  auto work = [&]() {
    for (;;) {
      const size_t index = next.fetch_add(1);
      if (index >= count || bad_kind.load() != 0) return;
      const PlannedTensor& t = file->tensors[index];
      const unsigned char* bytes = file->base + t.offset;
      int kind = 0;
      if (fnv1a(bytes, t.bytes, kFnvOffset) != file->checksums[index]) kind = 1;
      for (uint64_t at = 0; kind == 0 && at < t.bytes; at += 4)
        // all exponent bits set: infinity or NaN
        if ((little(bytes + at, 4) & 0x7f800000u) == 0x7f800000u) kind = 2;
      if (kind != 0) {
        int none = 0;
        if (bad_kind.compare_exchange_strong(none, kind)) bad_index.store(index);
        return;
      }
    }
  };
  const int workers = std::max(1, std::min<int>(threads, static_cast<int>(count)));
  std::vector<std::thread> pool;
  for (int i = 1; i < workers; ++i) pool.emplace_back(work);
  work();
  for (std::thread& thread : pool) thread.join();
  if (bad_kind.load() != 0) {
    const PlannedTensor& t = file->tensors[bad_index.load()];
    const std::string where = t.layer == kGlobalLayer
                                  ? std::string(role_name(t.role))
                                  : std::string(role_name(t.role)) + " of layer " +
                                        std::to_string(static_cast<int>(t.layer));
    return fail(HX_FILE_FORMAT, bad_kind.load() == 1 ? "%s: payload checksum mismatch"
                                                     : "%s contains a non-finite value",
                where.c_str());
  }
  return HX_FILE_OK;
}

}  // extern "C"
