// What this library needs from the engine's tiered expert residency
// (include/q4t/quant/moe_residency.h of the reference): the slot-mode weight layout
// (E = resident slots, include/q4t/quant/moe_weights.h:47-51) and the current
// expert -> slot table ON THE DEVICE.  The reference's MoEForward reads the selected ids
// back to the host, resolves them to slots (loading missing experts from the SSD tier) and
// writes slot ids back (src/model/moe.cu:495-909); that tier - eviction, loading, the
// sub-chunk planner - stays in the engine.  On B200 a whole layer's experts fit in HBM
// many times over, so the operator only consumes the table the tier publishes: an expert
// that is not resident (negative entry) contributes nothing to the token's sum.
#pragma once
#include <cstdint>

#include "q4t/quant/moe_weights.h"

namespace q4t::quant {

class MoEResidency {
 public:
  // layout: slot-mode weights (layout.E slots); device_slot_of_expert: device int32
  // [experts], entry e = slot holding expert e, or negative.
  MoEResidency(const MoEWeightLayout& layout, const int32_t* device_slot_of_expert, int experts)
      : layout_(layout), table_(device_slot_of_expert), experts_(experts) {}
  const MoEWeightLayout& Layout() const { return layout_; }
  int Slots() const { return layout_.E; }
  int Experts() const { return experts_; }
  const int32_t* DeviceSlotOfExpert() const { return table_; }

 private:
  MoEWeightLayout layout_;
  const int32_t* table_;
  int experts_;
};

}  // namespace q4t::quant
