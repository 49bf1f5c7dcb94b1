// TEST INFRASTRUCTURE.  Stand-in for the parallel-hashmap library's header, which the reference's
// engine headers include (include/mcts/phmap_transposition_table.h:12, node_tracker.h:9,
// transposition_table.h:12) and which is not available here.  Only enough for those HEADERS to
// compile, so that the adapter checks can use the reference's own MCTSSettings / MCTSStats /
// SearchResult types; none of the reference code that uses the maps is built.
#pragma once
#include <cstddef>
#include <functional>
#include <memory>
#include <unordered_map>
#include <unordered_set>
#include <utility>

namespace phmap {
struct NullMutex {};
namespace priv {
template <class K> using hash_default_hash = std::hash<K>;
template <class K> using hash_default_eq = std::equal_to<K>;
template <class T> using Allocator = std::allocator<T>;
}  // namespace priv
template <class K, class V, class H = std::hash<K>, class E = std::equal_to<K>,
          class A = std::allocator<std::pair<const K, V>>, size_t N = 4, class M = NullMutex>
class parallel_flat_hash_map : public std::unordered_map<K, V, H, E, A> {};
template <class K, class V, class H = std::hash<K>, class E = std::equal_to<K>,
          class A = std::allocator<std::pair<const K, V>>, size_t N = 4, class M = NullMutex>
class parallel_node_hash_map : public std::unordered_map<K, V, H, E, A> {};
template <class K, class V, class H = std::hash<K>, class E = std::equal_to<K>, class A = std::allocator<std::pair<const K, V>>>
class flat_hash_map : public std::unordered_map<K, V, H, E, A> {};
template <class K, class V, class H = std::hash<K>, class E = std::equal_to<K>, class A = std::allocator<std::pair<const K, V>>>
class node_hash_map : public std::unordered_map<K, V, H, E, A> {};
template <class K, class H = std::hash<K>, class E = std::equal_to<K>, class A = std::allocator<K>>
class flat_hash_set : public std::unordered_set<K, H, E, A> {};
}  // namespace phmap
