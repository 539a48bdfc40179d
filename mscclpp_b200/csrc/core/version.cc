#include <mscclpp/core.hpp>

namespace mscclpp {
std::string version() { return "0.9.0+b200.1"; }
}  // namespace mscclpp
