// slot_store.hpp — the on-disk form of KV that survives a restart: fixed-size slots in one file and a record
// file beside it, byte for byte the reference's format (runtime/model/SlotFile.cpp:238-323,398-438):
//   record file = 4096-byte header area { "SPLASHSF", version 1, label bytes, slot bytes, tag bytes, CRC-32C of
//   header + tag } + tag, then one record per slot index, each rounded up to 64 bytes:
//   { magic 0x53524543, payload CRC-32C, payload bytes } + label + CRC-32C of all of that;
//   an all-zero record is a free slot. Fields are little-endian as the host lays them out.
// A file written for another tag, slot size or label size is emptied when it opens; a record counts only while
// its slot lies wholly inside the slot file; a damaged record is a free slot.
// Labels are the reference's (runtime/engine/cache/DiskLabels.hpp:22-37).
//
// The reference's SlotFile is also an asynchronous IO worker with a disk quota; here the eviction tier is pinned
// host memory, so the store only has to seal that tier's slots to disk and bring them back: synchronous
// pread/pwrite, blocks returned with a hole punch where the file system has one.
#pragma once

#include <array>
#include <cstdint>
#include <optional>
#include <set>
#include <span>
#include <string>
#include <vector>

namespace rkb::model {

struct KvBlockLabel final {
  uint64_t id = 0;
  uint64_t parent = 0;
  uint64_t lastUsed = 0;
  uint64_t imagesLo = 0;
  uint64_t imagesHi = 0;
  std::array<uint32_t, 32> tokens{};
};
struct StateLabel final {
  uint64_t block = 0;
  uint64_t lastUsed = 0;
  uint32_t tokens = 0;
  uint32_t checkpoint = 0;
};
static_assert(sizeof(KvBlockLabel) == 168 && sizeof(StateLabel) == 24);

struct SlotRecord final {
  uint32_t index = 0;
  uint64_t payloadBytes = 0;
  uint32_t checksum = 0;
  std::vector<uint8_t> label;
};

constexpr uint64_t kRecordsHeaderBytes = 4096;
uint64_t recordBytesFor(uint32_t labelBytes) noexcept;
// The header and the tag after it; its checksum covers both.
std::vector<uint8_t> encodeRecordsHeader(uint64_t slotBytes, uint32_t labelBytes, std::span<const uint8_t> tag);
std::vector<uint8_t> encodeRecord(uint64_t recordBytes, uint64_t payloadBytes, uint32_t payloadChecksum, std::span<const uint8_t> label);
std::optional<SlotRecord> decodeRecord(std::span<const uint8_t> record, uint32_t index, uint32_t labelBytes, uint64_t slotBytes);

class SlotStore final {
public:
  struct Persistence final {
    std::string slots, records;
    std::vector<uint8_t> tag;
    uint32_t labelBytes = 0;
  };
  SlotStore(uint64_t slotBytes, const Persistence &persistence);
  ~SlotStore();
  SlotStore(const SlotStore &) = delete;
  SlotStore &operator=(const SlotStore &) = delete;

  uint64_t slotBytes() const noexcept { return slotBytes_; }
  uint32_t labelBytes() const noexcept { return labelBytes_; }
  // The slots an earlier process left, as read when the file opened.
  const std::vector<SlotRecord> &records() const noexcept { return records_; }
  // Stores the payload from the start of the slot and zeros the rest, then writes the record: a record never names
  // bytes that were not handed to the file. Only synchronize() makes either durable; a record that reached the
  // drive without its payload fails the payload checksum when it is adopted. False on an IO failure: the slot then
  // has no record.
  bool write(uint32_t index, std::span<const uint8_t> payload, uint32_t checksum, std::span<const uint8_t> label);
  bool read(uint32_t index, std::span<uint8_t> destination) const;
  // Clears the slot's record, then returns its blocks to the volume.
  bool free(uint32_t index);
  // Frees every recorded slot: the store is empty afterwards.
  bool clear();
  // The indices that hold a record now (those found at opening and those written since, minus those freed).
  const std::set<uint32_t> &recorded() const noexcept { return recorded_; }
  // Flushes slots and records to the drive.
  bool synchronize();

private:
  uint64_t slotBytes_;
  uint32_t labelBytes_ = 0;
  uint64_t recordBytes_ = 0;
  int slots_ = -1, recordsFile_ = -1;
  std::vector<SlotRecord> records_;
  std::set<uint32_t> recorded_;
  std::vector<uint8_t> zeros_;
};

} // namespace rkb::model
