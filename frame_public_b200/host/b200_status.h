// Shared by the adapter translation units: C ABI status -> frame::Status.
#pragma once

#include <string_view>

#include <frame/core/status.h>

namespace frame_b200 {

// Maps an fb200_status (same numbering as frame::ErrorCode) to a Status whose message is
// "<where>: <fb200_last_error()>".
frame::Status to_status(int rc, std::string_view where);

}  // namespace frame_b200
