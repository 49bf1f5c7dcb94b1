/* Build stub for the oracle/_ref recipe only: shadows the reference header of
 * the same name, which pulls in the engine and parallel-hashmap (absent).
 * src/mcts/mcts_node.cpp includes it but uses nothing from it. */
