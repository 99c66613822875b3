// Reader of the 26B-A4B weight artifact container (G4A4MIX1 / G4A4BF16): memory-maps the file,
// checks its header, its entry table and the global scales of every quantised entry when it is
// opened, and on request every payload byte (padding, scale codes, per-tensor and whole-payload
// SHA-256) -- ArtifactFile::Open / ValidateMetadata / VerifyFull of the reference
// (src/models/gemma4/26b_a4b/artifact.cc:64-221, include/gewell/models/gemma4/26b_a4b/artifact.h).
//
// Layout (little endian): a 4096-byte header -- magic, ten 32-bit geometry fields, five 64-bit sizes
// at 48..87, the tied-head alias at 88..95, zeros to 167, SHA-256 digests of the configuration (168),
// the source index (200), the entry table (232), the payload (264) and the header itself with that
// field zeroed (296) -- then one 72-byte entry per tensor of the inventory, zero padding to the next
// 4096-byte boundary, and the tensors' payloads, each padded with zeros to 4096 bytes.
//
// The reference compiles its inventory (12,117 tensors of the whole model) into the reader; here the
// caller passes it, so that the reader serves any model of this container family.  Host code only.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

using namespace gw;

namespace {

constexpr uint64_t kHeaderBytes = 4096, kEntryBytes = 72, kAlignment = 4096;

uint64_t align_to(uint64_t value, uint64_t alignment) { return (value + alignment - 1) / alignment * alignment; }

uint64_t little_endian(const uint8_t* bytes, unsigned width) {
  uint64_t value = 0;
  for (unsigned i = 0; i < width; ++i) value |= uint64_t(bytes[i]) << (8 * i);
  return value;
}

bool all_zero(const uint8_t* data, uint64_t size) {
  for (uint64_t i = 0; i < size; ++i)
    if (data[i] != 0) return false;
  return true;
}

// SHA-256 (FIPS 180-4), incremental.
class Sha256 {
 public:
  Sha256() {
    static const uint32_t initial[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
                                        0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    std::memcpy(state_, initial, sizeof(state_));
  }
  void add(const uint8_t* data, uint64_t size) {
    total_ += size;
    while (size > 0) {
      const uint64_t take = std::min<uint64_t>(size, 64 - fill_);
      std::memcpy(block_ + fill_, data, take);
      fill_ += unsigned(take);
      data += take;
      size -= take;
      if (fill_ == 64) {
        compress(block_);
        fill_ = 0;
      }
    }
  }
  void finish(uint8_t digest[32]) {
    const uint64_t bits = total_ * 8;
    const uint8_t one = 0x80, zero = 0;
    add(&one, 1);
    while (fill_ != 56) add(&zero, 1);
    uint8_t length[8];
    for (int i = 0; i < 8; ++i) length[i] = uint8_t(bits >> (56 - 8 * i));
    add(length, 8);
    for (int i = 0; i < 8; ++i)
      for (int b = 0; b < 4; ++b) digest[4 * i + b] = uint8_t(state_[i] >> (24 - 8 * b));
  }

 private:
  static uint32_t rotate(uint32_t x, unsigned n) { return (x >> n) | (x << (32 - n)); }
  void compress(const uint8_t* block) {
    static const uint32_t k[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = uint32_t(block[4 * i]) << 24 | uint32_t(block[4 * i + 1]) << 16 | uint32_t(block[4 * i + 2]) << 8 | block[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotate(w[i - 15], 7) ^ rotate(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotate(w[i - 2], 17) ^ rotate(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = state_[0], b = state_[1], c = state_[2], d = state_[3], e = state_[4], f = state_[5], g = state_[6], h = state_[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = h + (rotate(e, 6) ^ rotate(e, 11) ^ rotate(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
      const uint32_t t2 = (rotate(a, 2) ^ rotate(a, 13) ^ rotate(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    state_[0] += a; state_[1] += b; state_[2] += c; state_[3] += d;
    state_[4] += e; state_[5] += f; state_[6] += g; state_[7] += h;
  }
  uint32_t state_[8];
  uint8_t block_[64];
  unsigned fill_ = 0;
  uint64_t total_ = 0;
};

bool digest_equals(const uint8_t* data, uint64_t size, const uint8_t* expected) {
  Sha256 hash;
  hash.add(data, size);
  uint8_t digest[32];
  hash.finish(digest);
  return std::memcmp(digest, expected, 32) == 0;
}

}  // namespace

struct gw_artifact {
  int fd = -1;
  const uint8_t* data = nullptr;
  size_t size = 0;
  bool mixed = false;
  std::vector<gw_artifact_tensor_spec> inventory;
  std::vector<gw_artifact_entry> entries;
  uint64_t data_offset = 0;
  ~gw_artifact() {
    if (data) munmap(const_cast<uint8_t*>(data), size);
    if (fd >= 0) close(fd);
  }
};

namespace {

// tensor_bytes (artifact.cc:64-71)
uint64_t entry_bytes(const gw_artifact_tensor_spec& spec, uint32_t storage) {
  const uint64_t elements = uint64_t(spec.rows) * (spec.rank == 1 ? 1 : spec.columns);
  if (storage == GW_STORAGE_BF16) return elements * 2;
  return gw_projection_entry_bytes(storage, spec.rows, spec.columns);
}

// ValidateMetadata (artifact.cc:149-190)
gw_status validate_metadata(gw_artifact& a) {
  const uint8_t* d = a.data;
  const uint64_t count = a.inventory.size();
  a.mixed = std::memcmp(d, "G4A4MIX1", 8) == 0;
  if (!a.mixed && std::memcmp(d, "G4A4BF16", 8) != 0) return fail(GW_INVALID_ARGUMENT, "wrong 26B artifact identity");
  const uint64_t geometry[10] = {1, kHeaderBytes, kEntryBytes, count, count + 1, 1, kAlignment, 1, 1, 1};
  for (unsigned i = 0; i < 10; ++i)
    if (little_endian(d + 8 + 4 * i, 4) != geometry[i]) return fail(GW_INVALID_ARGUMENT, "invalid 26B header geometry");
  // the output head is an alias of the embedding: logical id = tensor count, physical id 0
  if (little_endian(d + 88, 4) != count || little_endian(d + 92, 4) != 0) return fail(GW_INVALID_ARGUMENT, "invalid 26B tied-head alias");
  if (!all_zero(d + 96, 72) || !all_zero(d + 328, kHeaderBytes - 328))
    return fail(GW_INVALID_ARGUMENT, "nonzero 26B header reserved bytes");
  std::vector<uint8_t> header(d, d + kHeaderBytes);
  std::fill_n(header.begin() + 296, 32, uint8_t(0));
  if (!digest_equals(header.data(), header.size(), d + 296)) return fail(GW_INVALID_ARGUMENT, "26B header checksum mismatch");
  if (!digest_equals(d + kHeaderBytes, count * kEntryBytes, d + 232))
    return fail(GW_INVALID_ARGUMENT, "26B entry table checksum mismatch");
  uint64_t offset = a.data_offset, logical_bytes = 0;
  a.entries.reserve(count);
  for (uint64_t i = 0; i < count; ++i) {
    const gw_artifact_tensor_spec& spec = a.inventory[i];
    const uint8_t* entry = d + kHeaderBytes + i * kEntryBytes;
    const uint32_t storage = entry[7];
    if (storage > 2 || (!a.mixed && storage != 0)) return fail(GW_INVALID_ARGUMENT, "invalid 26B storage type");
    if (storage != GW_STORAGE_BF16 && !spec.projection) return fail(GW_INVALID_ARGUMENT, "quantized 26B tensor is not a projection");
    const uint64_t bytes = entry_bytes(spec, storage);
    if (little_endian(entry, 2) != i || little_endian(entry + 2, 2) != uint16_t(int16_t(spec.layer)) ||
        little_endian(entry + 4, 2) != spec.role || entry[6] != spec.rank || little_endian(entry + 8, 4) != spec.rows ||
        little_endian(entry + 12, 4) != (spec.rank == 1 ? 0 : spec.columns) || little_endian(entry + 16, 4) != 0 ||
        little_endian(entry + 20, 8) != offset || little_endian(entry + 28, 8) != bytes || !all_zero(entry + 68, 4))
      return fail(GW_INVALID_ARGUMENT, "invalid 26B tensor entry " + std::to_string(i));
    gw_artifact_entry e{};
    e.offset = offset;
    e.bytes = bytes;
    e.storage = storage;
    std::memcpy(e.sha256, entry + 36, 32);
    e.data = nullptr;            // set once the file size is known to cover it
    a.entries.push_back(e);
    offset += align_to(bytes, kAlignment);
    logical_bytes += bytes;
  }
  if (little_endian(d + 48, 8) != kHeaderBytes || little_endian(d + 56, 8) != a.data_offset ||
      little_endian(d + 64, 8) != logical_bytes || little_endian(d + 72, 8) != offset - a.data_offset ||
      little_endian(d + 80, 8) != offset || a.size != offset)
    return fail(GW_INVALID_ARGUMENT, "invalid 26B artifact size");
  for (gw_artifact_entry& e : a.entries) {
    e.data = d + e.offset;
    if (e.storage == GW_STORAGE_BF16) continue;
    float weight, input;
    std::memcpy(&weight, e.data + e.bytes - 8, 4);
    std::memcpy(&input, e.data + e.bytes - 4, 4);
    if (!(std::isfinite(weight) && weight > 0 && std::isfinite(input) && input > 0 && std::isfinite(1.0F / input) &&
          std::isfinite(weight * input) && weight * input > 0))
      return fail(GW_INVALID_ARGUMENT, "invalid 26B global scales");
  }
  return GW_OK;
}

}  // namespace

extern "C" {

gw_status gw_artifact_open(const char* path, const gw_artifact_tensor_spec* inventory, uint32_t count, gw_artifact** artifact) {
  clear_error();
  if (!path || !inventory || count == 0 || !artifact) return fail(GW_INVALID_ARGUMENT, "artifact open requires a path and an inventory");
  auto a = std::unique_ptr<gw_artifact>(new (std::nothrow) gw_artifact());
  if (!a) return fail(GW_CUDA_ERROR, "out of host memory");
  a->inventory.assign(inventory, inventory + count);
  a->data_offset = align_to(kHeaderBytes + uint64_t(count) * kEntryBytes, kAlignment);
  a->fd = open(path, O_RDONLY | O_CLOEXEC);
  if (a->fd < 0) return fail(GW_INVALID_ARGUMENT, "cannot open 26B artifact");
  struct stat status {};
  if (fstat(a->fd, &status) != 0 || !S_ISREG(status.st_mode) || uint64_t(status.st_size) < a->data_offset)
    return fail(GW_INVALID_ARGUMENT, "truncated 26B artifact");
  a->size = size_t(status.st_size);
  void* mapping = mmap(nullptr, a->size, PROT_READ, MAP_PRIVATE, a->fd, 0);
  if (mapping == MAP_FAILED) return fail(GW_INVALID_ARGUMENT, "cannot map 26B artifact");
  a->data = static_cast<const uint8_t*>(mapping);
  const gw_status checked = validate_metadata(*a);
  if (checked != GW_OK) return checked;
  *artifact = a.release();
  return GW_OK;
}

void gw_artifact_close(gw_artifact* artifact) { delete artifact; }

uint32_t gw_artifact_count(const gw_artifact* a) { return a ? uint32_t(a->entries.size()) : 0; }
int gw_artifact_is_mixed(const gw_artifact* a) { return a && a->mixed ? 1 : 0; }
uint64_t gw_artifact_file_bytes(const gw_artifact* a) { return a ? a->size : 0; }

gw_status gw_artifact_entry_at(const gw_artifact* a, uint32_t id, gw_artifact_entry* entry) {
  clear_error();
  if (!a || !entry || id >= a->entries.size()) return fail(GW_INVALID_ARGUMENT, "no such 26B artifact entry");
  *entry = a->entries[id];
  return GW_OK;
}

// VerifyFull (artifact.cc:194-221)
gw_status gw_artifact_verify_full(const gw_artifact* a) {
  clear_error();
  if (!a || !a->data) return fail(GW_INVALID_ARGUMENT, "26B artifact is not open");
  const uint64_t table_end = kHeaderBytes + a->entries.size() * kEntryBytes;
  if (!all_zero(a->data + table_end, a->data_offset - table_end)) return fail(GW_INVALID_ARGUMENT, "nonzero 26B table padding");
  Sha256 payload;
  for (size_t i = 0; i < a->entries.size(); ++i) {
    const gw_artifact_entry& e = a->entries[i];
    const gw_artifact_tensor_spec& spec = a->inventory[i];
    if (e.storage != GW_STORAGE_BF16) {
      const gw_status checked = gw_validate_projection_entry(e.storage, spec.rows, spec.columns, e.data, e.bytes);
      if (checked != GW_OK) return checked;
    }
    if (!digest_equals(e.data, e.bytes, e.sha256)) return fail(GW_INVALID_ARGUMENT, "26B tensor checksum mismatch");
    const uint64_t padded = align_to(e.bytes, kAlignment);
    if (!all_zero(e.data + e.bytes, padded - e.bytes)) return fail(GW_INVALID_ARGUMENT, "nonzero 26B tensor padding");
    payload.add(e.data, padded);
  }
  uint8_t digest[32];
  payload.finish(digest);
  if (std::memcmp(digest, a->data + 264, 32) != 0) return fail(GW_INVALID_ARGUMENT, "26B payload checksum mismatch");
  return GW_OK;
}

}  // extern "C"
