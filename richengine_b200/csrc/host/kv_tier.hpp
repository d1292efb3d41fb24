// kv_tier.hpp — the eviction tier as the cache drives it, and its pinned-host implementation.
//
// Interface after engine::KvTier / KvTransfer / KvDiskSlot (runtime/engine/cache/KvTier.hpp:13-63):
// a page stays valid until its demotion reports success; no command writes a page being demoted or
// touches a page being restored. The slot store here is pinned host memory (rk_tier_*, capi.cu)
// instead of the reference's SSD slot file (runtime/engine/cache/KvPageTier.cpp).
#pragma once

#include "../../../include/richkv.h"

#include <cstdint>
#include <memory>
#include <stdexcept>

namespace rkb::engine {

// One slot of the tier; releasing the last handle frees the slot.
class KvTierSlot {
public:
  virtual ~KvTierSlot() = default;
};

class KvTransfer {
public:
  virtual ~KvTransfer() = default;
  virtual bool ready() const noexcept = 0;
  virtual bool finish() = 0; // true = the copy landed
};

class KvTier {
public:
  virtual ~KvTier() = default;
  virtual uint64_t slotBytes() const noexcept = 0;
  virtual bool writable() const noexcept = 0;
  virtual bool canDemote() const noexcept = 0;
  virtual bool canRestore() const noexcept = 0;
  virtual std::shared_ptr<KvTierSlot> acquireSlot() = 0; // null when the quota is full
  virtual std::unique_ptr<KvTransfer> demote(uint32_t page, std::shared_ptr<KvTierSlot> slot) = 0;  // null = not now
  virtual std::unique_ptr<KvTransfer> restore(std::shared_ptr<KvTierSlot> slot, uint32_t page) = 0; // null = not now
  virtual void poll() = 0;
  // Persistence (engine::KvTier::persistent / label, KvPageTier::adopt: runtime/engine/cache/KvTier.hpp:40-47,
  // runtime/engine/cache/KvPageTier.hpp:38-43). A tier that can be sealed to a slot store exposes the host bytes
  // of a landed slot with the CRC-32C taken when the page was packed, and takes a recorded payload back into a
  // slot of its own whose first restore is checked against the record.
  struct SlotPayload { const void *bytes = nullptr; uint64_t size = 0; uint32_t checksum = 0; };
  virtual bool slotPayload(const KvTierSlot &, SlotPayload *) const { return false; }
  virtual std::shared_ptr<KvTierSlot> adoptSlot(const void *, uint64_t, uint32_t) { return {}; }
};

// Pinned-host tier over the C ABI.
class HostKvTier final : public KvTier {
public:
  HostKvTier(void *storage, uint32_t slots, uint32_t transfers, void *computeStream = nullptr)
      : tier_(rk_tier_create(storage, slots, transfers)), stream_(computeStream) {
    if (!tier_) throw std::runtime_error(rk_last_error());
  }
  ~HostKvTier() override { rk_tier_destroy(tier_); }
  HostKvTier(const HostKvTier &) = delete;
  HostKvTier &operator=(const HostKvTier &) = delete;

  uint64_t slotBytes() const noexcept override { return rk_tier_slot_bytes(tier_); }
  bool writable() const noexcept override { return rk_tier_writable(tier_) != 0; }
  bool canDemote() const noexcept override { return rk_tier_can_demote(tier_) != 0; }
  bool canRestore() const noexcept override { return rk_tier_can_restore(tier_) != 0; }
  std::shared_ptr<KvTierSlot> acquireSlot() override {
    const int64_t id = rk_tier_acquire_slot(tier_);
    if (id < 0) return {};
    return std::make_shared<Slot>(tier_, uint32_t(id));
  }
  std::unique_ptr<KvTransfer> demote(uint32_t page, std::shared_ptr<KvTierSlot> slot) override {
    auto held = std::dynamic_pointer_cast<Slot>(slot);
    if (!held) throw std::invalid_argument("KV tier slot belongs to another tier");
    const int id = rk_tier_demote(tier_, page, held->id, stream_);
    if (id < 0) return {};
    return std::make_unique<Ticket>(tier_, uint32_t(id), std::move(held));
  }
  std::unique_ptr<KvTransfer> restore(std::shared_ptr<KvTierSlot> slot, uint32_t page) override {
    auto held = std::dynamic_pointer_cast<Slot>(slot);
    if (!held) throw std::invalid_argument("KV tier slot belongs to another tier");
    const int id = rk_tier_restore(tier_, held->id, page, stream_);
    if (id < 0) return {};
    return std::make_unique<Ticket>(tier_, uint32_t(id), std::move(held));
  }
  void poll() override { rk_tier_poll(tier_); }
  bool slotPayload(const KvTierSlot &slot, SlotPayload *out) const override {
    const auto *held = dynamic_cast<const Slot *>(&slot);
    if (!held) return false;
    *out = {rk_tier_slot_host_pointer(tier_, held->id), rk_tier_slot_bytes(tier_), rk_tier_slot_checksum(tier_, held->id)};
    return out->bytes != nullptr;
  }
  std::shared_ptr<KvTierSlot> adoptSlot(const void *payload, uint64_t bytes, uint32_t checksum) override {
    const int64_t id = rk_tier_adopt_slot(tier_, payload, bytes, checksum);
    if (id < 0) return {};
    return std::make_shared<Slot>(tier_, uint32_t(id));
  }
  void *handle() const noexcept { return tier_; }
  void failNext(uint32_t count) { rk_tier_fail_next(tier_, count); }

private:
  struct Slot final : KvTierSlot {
    Slot(void *tier, uint32_t slot) : tier(tier), id(slot) {}
    ~Slot() override { rk_tier_release_slot(tier, id); }
    void *tier;
    uint32_t id;
  };
  class Ticket final : public KvTransfer {
  public:
    Ticket(void *tier, uint32_t id, std::shared_ptr<Slot> slot) : tier_(tier), id_(id), slot_(std::move(slot)) {}
    ~Ticket() override {
      if (!finished_) { // never leave a transfer id occupied
        while (!rk_tier_transfer_ready(tier_, id_)) rk_tier_drain(tier_);
        rk_tier_transfer_finish(tier_, id_);
      }
    }
    bool ready() const noexcept override { return finished_ || rk_tier_transfer_ready(tier_, id_) != 0; }
    bool finish() override {
      if (!finished_) {
        success_ = rk_tier_transfer_finish(tier_, id_) == 1;
        finished_ = true;
      }
      return success_;
    }

  private:
    void *tier_;
    uint32_t id_;
    std::shared_ptr<Slot> slot_;
    bool finished_ = false, success_ = false;
  };

  void *tier_;
  void *stream_;
};

} // namespace rkb::engine
