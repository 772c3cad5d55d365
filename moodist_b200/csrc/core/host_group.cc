#include "host_group.h"

#include "log.h"

namespace moodist {
std::unique_ptr<HostGroup> HostGroup::create(KVStore&, const std::string&, int, int) {
  fail("moodist: the host engine is not built in this snapshot");
}
}  // namespace moodist
