// Status codes of the operator surface. Mirrors Catlass::Status (include/catlass/status.hpp:16-20).
#pragma once

namespace Catlass {

enum class Status {
    kSuccess = 0,
    kInvalid = 1,
};

}  // namespace Catlass
