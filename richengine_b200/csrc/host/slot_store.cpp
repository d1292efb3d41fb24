// slot_store.cpp — record and slot files of the persistent tier (format: slot_store.hpp).
#include "slot_store.hpp"

#include "../../../include/richkv.h"

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <limits>
#include <stdexcept>
#include <sys/stat.h>
#include <system_error>
#include <unistd.h>

namespace rkb::model {
namespace {

constexpr char kRecordsMagic[8] = {'S', 'P', 'L', 'A', 'S', 'H', 'S', 'F'};
constexpr uint32_t kRecordsVersion = 1;
constexpr uint32_t kRecordMagic = 0x53524543;

struct RecordsHeader final {
  char magic[8];
  uint32_t version;
  uint32_t labelBytes;
  uint64_t slotBytes;
  uint32_t tagBytes;
  uint32_t checksum;
};
struct RecordHead final {
  uint32_t magic;
  uint32_t payloadChecksum;
  uint64_t payloadBytes;
};
static_assert(sizeof(RecordsHeader) == 32 && sizeof(RecordHead) == 16);

uint32_t crc(std::span<const uint8_t> bytes) { return rk_crc32c_host(bytes.data(), bytes.size(), 0); }

bool writeAll(int descriptor, const uint8_t *data, size_t size, off_t offset) {
  while (size) {
    const ssize_t moved = ::pwrite(descriptor, data, size, offset);
    if (moved < 0 && errno == EINTR) continue;
    if (moved <= 0) return false;
    data += moved; size -= size_t(moved); offset += moved;
  }
  return true;
}
bool readAll(int descriptor, uint8_t *data, size_t size, off_t offset) {
  while (size) {
    const ssize_t moved = ::pread(descriptor, data, size, offset);
    if (moved < 0 && errno == EINTR) continue;
    if (moved <= 0) return false; // a short file is a failed read
    data += moved; size -= size_t(moved); offset += moved;
  }
  return true;
}
uint64_t fileBytes(int descriptor, const char *what) {
  struct stat status {};
  if (::fstat(descriptor, &status) < 0) throw std::system_error(errno, std::generic_category(), what);
  return uint64_t(status.st_size);
}
int openFile(const std::string &path, const char *what) {
  const int descriptor = ::open(path.c_str(), O_RDWR | O_CREAT | O_CLOEXEC | O_NOFOLLOW, 0600);
  if (descriptor < 0) throw std::system_error(errno, std::generic_category(), what);
  return descriptor;
}

} // namespace

uint64_t recordBytesFor(uint32_t labelBytes) noexcept {
  const uint64_t bytes = sizeof(RecordHead) + uint64_t(labelBytes) + sizeof(uint32_t);
  return (bytes + 63) / 64 * 64;
}

std::vector<uint8_t> encodeRecordsHeader(uint64_t slotBytes, uint32_t labelBytes, std::span<const uint8_t> tag) {
  if (sizeof(RecordsHeader) + tag.size() > kRecordsHeaderBytes) throw std::invalid_argument("slot file tag is too long");
  RecordsHeader header{};
  std::memcpy(header.magic, kRecordsMagic, sizeof(header.magic));
  header.version = kRecordsVersion;
  header.labelBytes = labelBytes;
  header.slotBytes = slotBytes;
  header.tagBytes = uint32_t(tag.size());
  std::vector<uint8_t> bytes(sizeof(header) + tag.size());
  std::memcpy(bytes.data(), &header, sizeof(header));
  if (!tag.empty()) std::memcpy(bytes.data() + sizeof(header), tag.data(), tag.size());
  header.checksum = crc(bytes); // over the header with a zero checksum field, and the tag
  std::memcpy(bytes.data(), &header, sizeof(header));
  return bytes;
}

std::vector<uint8_t> encodeRecord(uint64_t recordBytes, uint64_t payloadBytes, uint32_t payloadChecksum, std::span<const uint8_t> label) {
  const size_t covered = sizeof(RecordHead) + label.size();
  if (covered + sizeof(uint32_t) > recordBytes) throw std::invalid_argument("slot record is too short for its label");
  std::vector<uint8_t> record(recordBytes);
  const RecordHead head{kRecordMagic, payloadChecksum, payloadBytes};
  std::memcpy(record.data(), &head, sizeof(head));
  if (!label.empty()) std::memcpy(record.data() + sizeof(head), label.data(), label.size());
  const uint32_t checksum = crc(std::span<const uint8_t>(record).first(covered));
  std::memcpy(record.data() + covered, &checksum, sizeof(checksum));
  return record;
}

std::optional<SlotRecord> decodeRecord(std::span<const uint8_t> record, uint32_t index, uint32_t labelBytes, uint64_t slotBytes) {
  const size_t covered = sizeof(RecordHead) + labelBytes;
  if (record.size() < covered + sizeof(uint32_t)) return std::nullopt;
  RecordHead head;
  std::memcpy(&head, record.data(), sizeof(head));
  if (head.magic != kRecordMagic || !head.payloadBytes || head.payloadBytes > slotBytes) return std::nullopt;
  uint32_t checksum;
  std::memcpy(&checksum, record.data() + covered, sizeof(checksum));
  if (checksum != crc(record.first(covered))) return std::nullopt;
  const auto label = record.subspan(sizeof(head), labelBytes);
  return SlotRecord{index, head.payloadBytes, head.payloadChecksum, {label.begin(), label.end()}};
}

SlotStore::SlotStore(uint64_t slotBytes, const Persistence &persistence) : slotBytes_(slotBytes) {
  if (!slotBytes || slotBytes % 4096) throw std::invalid_argument("a slot is a whole number of host pages");
  if (!persistence.labelBytes) throw std::invalid_argument("a persistent slot file needs a label size");
  labelBytes_ = persistence.labelBytes;
  recordBytes_ = recordBytesFor(labelBytes_);
  const std::vector<uint8_t> header = encodeRecordsHeader(slotBytes_, labelBytes_, persistence.tag);
  slots_ = openFile(persistence.slots, "open slot file");
  try {
    recordsFile_ = openFile(persistence.records, "open slot record file");
    const uint64_t recordFileBytes = fileBytes(recordsFile_, "stat slot record file");
    std::vector<uint8_t> found(header.size());
    if (recordFileBytes < kRecordsHeaderBytes || !readAll(recordsFile_, found.data(), found.size(), 0) || found != header) {
      // Written for something else, or new: start empty.
      if (::ftruncate(slots_, 0) < 0 || ::ftruncate(recordsFile_, 0) < 0 || !writeAll(recordsFile_, header.data(), header.size(), 0) ||
          ::ftruncate(recordsFile_, off_t(kRecordsHeaderBytes)) < 0)
        throw std::system_error(errno, std::generic_category(), "reset slot file");
      return;
    }
    // A record counts only while its slot lies wholly inside the slot file.
    const uint64_t slots = fileBytes(slots_, "stat slot file") / slotBytes_;
    const uint64_t recorded = (recordFileBytes - kRecordsHeaderBytes) / recordBytes_;
    if (std::max(slots, recorded) > std::numeric_limits<uint32_t>::max()) throw std::runtime_error("slot file holds more slots than it can index");
    std::vector<uint8_t> records(std::min(slots, recorded) * recordBytes_);
    if (!records.empty() && !readAll(recordsFile_, records.data(), records.size(), off_t(kRecordsHeaderBytes)))
      throw std::system_error(errno, std::generic_category(), "read slot records");
    for (uint64_t index = 0; index < records.size() / recordBytes_; ++index) {
      const auto record = std::span<const uint8_t>(records).subspan(index * recordBytes_, recordBytes_);
      if (auto slot = decodeRecord(record, uint32_t(index), labelBytes_, slotBytes_)) {
        recorded_.insert(slot->index);
        records_.push_back(std::move(*slot));
      }
    }
  } catch (...) {
    if (recordsFile_ >= 0) ::close(recordsFile_);
    ::close(slots_);
    throw;
  }
}

SlotStore::~SlotStore() {
  if (recordsFile_ >= 0) ::close(recordsFile_);
  if (slots_ >= 0) ::close(slots_);
}

bool SlotStore::write(uint32_t index, std::span<const uint8_t> payload, uint32_t checksum, std::span<const uint8_t> label) {
  if (payload.empty() || payload.size() > slotBytes_ || label.size() != labelBytes_) throw std::invalid_argument("invalid slot write");
  const off_t at = off_t(uint64_t(index) * slotBytes_);
  if (!writeAll(slots_, payload.data(), payload.size(), at)) return false;
  if (payload.size() < slotBytes_) { // the rest of the slot is zeros
    if (zeros_.size() < slotBytes_ - payload.size()) zeros_.assign(slotBytes_ - payload.size(), 0);
    if (!writeAll(slots_, zeros_.data(), slotBytes_ - payload.size(), at + off_t(payload.size()))) return false;
  }
  // The record follows the slot's write: a record never names bytes that were not handed to the file.
  const std::vector<uint8_t> record = encodeRecord(recordBytes_, payload.size(), checksum, label);
  if (!writeAll(recordsFile_, record.data(), record.size(), off_t(kRecordsHeaderBytes + uint64_t(index) * recordBytes_))) return false;
  recorded_.insert(index);
  return true;
}

bool SlotStore::read(uint32_t index, std::span<uint8_t> destination) const {
  if (destination.size() > slotBytes_) throw std::invalid_argument("invalid slot read");
  return readAll(slots_, destination.data(), destination.size(), off_t(uint64_t(index) * slotBytes_));
}

bool SlotStore::free(uint32_t index) {
  // The record goes first: blocks that returned under a live record would read as a damaged payload.
  const std::vector<uint8_t> cleared(recordBytes_, 0);
  const off_t at = off_t(kRecordsHeaderBytes + uint64_t(index) * recordBytes_);
  if (uint64_t(at) + recordBytes_ <= fileBytes(recordsFile_, "stat slot record file") && !writeAll(recordsFile_, cleared.data(), cleared.size(), at))
    return false;
#ifdef FALLOC_FL_PUNCH_HOLE
  ::fallocate(slots_, FALLOC_FL_PUNCH_HOLE | FALLOC_FL_KEEP_SIZE, off_t(uint64_t(index) * slotBytes_), off_t(slotBytes_)); // best effort
#endif
  recorded_.erase(index);
  return true;
}

bool SlotStore::clear() {
  if (::ftruncate(slots_, 0) < 0 || ::ftruncate(recordsFile_, off_t(kRecordsHeaderBytes)) < 0) return false;
  records_.clear();
  recorded_.clear();
  return true;
}

bool SlotStore::synchronize() { return ::fdatasync(slots_) == 0 && ::fdatasync(recordsFile_) == 0; }

} // namespace rkb::model
