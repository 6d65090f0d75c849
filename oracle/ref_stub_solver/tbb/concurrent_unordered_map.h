/* Stand-in for a TBB header that is not installed here: the reference's solver source uses the
 * container in its MILP preparation; the parity pin never runs that code, and a plain
 * std::unordered_map is enough for it to compile.  Test infrastructure. */
#pragma once
#include <unordered_map>
namespace tbb {
template <typename K, typename V, typename H = std::hash<K>, typename E = std::equal_to<K>>
class concurrent_unordered_map : public std::unordered_map<K, V, H, E> {
 public:
  using std::unordered_map<K, V, H, E>::unordered_map;
};
}  // namespace tbb
