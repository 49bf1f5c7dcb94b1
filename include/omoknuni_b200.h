/* omoknuni_b200.h — C ABI of the B200 (sm_100a) leaf-parallel evaluation path.
 *
 * Plain C: opaque handles, plain pointers and sizes, int status returns
 * (0 = OK), no exceptions, no torch / libtorch types.  Every entry point cites
 * the interface of the reference project (cosmosapjw-quantum/omoknuni_small,
 * paths relative to that project's root) that it replaces.
 *
 * Two layers:
 *   ob200_launch_*  raw launchers over caller-owned DEVICE memory, asynchronous
 *                   on the given stream — the same shape as the reference's
 *                   `extern "C" launch*Kernel` functions.
 *   ob200_net_*     handle-based calls that own their device buffers and take
 *                   HOST buffers — what the reference's C++ classes bind
 *                   through the adapters in omoknuni_small_b200/adapter/.
 *
 * There is no CPU fallback: every call needs a CUDA device of compute
 * capability 10.x and returns OB200_ERR_NO_DEVICE otherwise.
 */
#ifndef OMOKNUNI_B200_H
#define OMOKNUNI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OB200_VERSION 2

/* Status codes. */
enum {
    OB200_OK = 0,
    OB200_ERR_INVALID = 1,     /* null pointer, bad size, bad enum            */
    OB200_ERR_NO_DEVICE = 2,   /* no CUDA device / not compute capability 10  */
    OB200_ERR_CUDA = 3,        /* a CUDA runtime call failed                  */
    OB200_ERR_STATE = 4,       /* call order (weights not finalised, ...)     */
    OB200_ERR_UNSUPPORTED = 5, /* shape outside what the kernels are built for*/
    OB200_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out          */
    OB200_ERR_TOO_LARGE = 7    /* size beyond a stated maximum                */
};

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer; NULL is the
 * legacy default stream. */
typedef void* ob200_stream;

/* Thread-local text of the last error raised by a call on this thread. */
const char* ob200_last_error(void);
int ob200_version(void);
/* Number of usable (compute capability 10.x) devices; 0 when none. */
int ob200_device_count(void);

/* ------------------------------------------------------------------------- *
 *  Tree statistics: structure of arrays over (node, child slot) edges.
 *
 *  Replaces the dense libtorch tensors of GPUBatchEvaluator::TreeTensors
 *  (include/mcts/gpu_batch_evaluator.h:116-133) and the per-child heap nodes
 *  of MCTSNode (include/mcts/mcts_node.h:160-198).  Row r of every edge array
 *  holds the child slots of node r; rows are `pitch` elements apart, pitch a
 *  multiple of 4 so that rows start on 16-byte boundaries; slots in
 *  [n_children, pitch) are padding and never selected.  Child slot order is
 *  the tie-break order (lowest slot wins).  N, W, P and VL must be 16-byte
 *  aligned (checked: OB200_ERR_INVALID otherwise); legal_bits needs 4-byte
 *  alignment only, but a 16-byte aligned mask array with mask_words a multiple of
 *  4 is what lets large launches take the fastest selection kernel.
 * ------------------------------------------------------------------------- */
typedef struct ob200_tree_view {
    int32_t* N;              /* [n_nodes][pitch] visit count of the child      */
    float* W;                /* [n_nodes][pitch] value sum of the child        */
    float* P;                /* [n_nodes][pitch] prior of the child            */
    int32_t* VL;             /* [n_nodes][pitch] virtual-loss counter          */
    uint32_t* legal_bits;    /* [n_nodes][mask_words] bit s = child slot s exists */
    int32_t* node_visits;    /* [n_nodes] visit count of the node itself       */
    int32_t* child_node;     /* [n_nodes][pitch] node id of the child, -1 = not
                                expanded; may be NULL for flat selection       */
    int32_t n_nodes;
    int32_t n_children;      /* child slots per node (225, 362, 4672, ...)     */
    int32_t pitch;           /* >= n_children, multiple of 4                   */
    int32_t mask_words;      /* >= ceil(n_children / 32)                       */
} ob200_tree_view;

/* pitch / mask_words the kernels expect for a given child count. */
int32_t ob200_tree_pitch(int32_t n_children);
int32_t ob200_tree_mask_words(int32_t n_children);

/* Batched PUCT child selection with virtual loss.
 * Replaces MCTSNode::selectChild (src/mcts/mcts_node.cpp:90-236) + the
 * applyVirtualLoss call that follows it in the search loop
 * (src/mcts/mcts_engine_batch_tree_simple.cpp:102-111), and the launchers
 * launchUCBKernel + launchPathSelectionKernel
 * (src/mcts/gpu_batch_evaluator.cpp:9-33).
 * For i in [0, n): node = node_ids ? node_ids[i] : i;
 *   sel_out[i] = argmax over existing child slots of
 *        q + u,  q = (N+VL > 0) ? (W - (float)VL) / (float)(N+VL) : 0
 *                u = (P * (c_puct * sqrtf((float)node_visits))) / (1 + (float)(N+VL))
 *   in IEEE fp32 with the reference's operation order; strict '>' so the
 *   lowest slot wins ties; -1 when the node has no child slot; when no score
 *   compares greater than -inf (all NaN / -inf) the least-visited slot, as
 *   the reference's fallback does.
 *   If apply_vl != 0 and vl_value > 0: atomically VL[node][sel] += vl_value.
 * Distinct entries of node_ids may repeat; each sees the table as it was when
 * it read it (entries of one launch are not ordered against each other).
 * Rows of more than 256 slots in large launches (every launch of rows of 1,024
 * slots or more) use 8 bytes of scratch per entry, which the library keeps per
 * (device, stream) and obtains with cudaMallocAsync when a launch needs more
 * than the stream has: make the first such launch of a stream outside stream
 * capture.  Launches of rows up to 256 slots allocate nothing. */
int ob200_launch_puct_select(const ob200_tree_view* tree, const int32_t* node_ids, int32_t n,
                             float c_puct, int32_t vl_value, int32_t apply_vl,
                             int32_t* sel_out, ob200_stream stream);

/* VL[node][sel] += vl_value for each i with sel[i] >= 0.
 * Replaces MCTSNode::addVirtualLoss(int) (src/mcts/mcts_node_virtual_loss.cpp:15-20)
 * and launchApplyVirtualLossKernelCuda (src/mcts/gpu_virtual_loss.cpp:10-20). */
int ob200_launch_vl_apply(const ob200_tree_view* tree, const int32_t* node_ids,
                          const int32_t* sel, int32_t n, int32_t vl_value, ob200_stream stream);

/* old = VL; VL -= vl_value; if (old < vl_value) VL = 0   (clamp at zero).
 * Replaces MCTSNode::removeVirtualLoss(int) (src/mcts/mcts_node_virtual_loss.cpp:32-42)
 * and launchRemoveVirtualLossKernelCuda (src/mcts/gpu_virtual_loss.cpp:22-32). */
int ob200_launch_vl_revert(const ob200_tree_view* tree, const int32_t* node_ids,
                           const int32_t* sel, int32_t n, int32_t vl_value, ob200_stream stream);

/* Backup along recorded paths.  paths[i][d] = (node, child slot) for
 * d in [0, path_len[i]), root first, layout [n][max_depth][2] as the
 * reference's selected_paths tensor.  Walking leaf -> root with
 * v = leaf_values[i]: the edge gets N += 1, W += v, "VL -= 1 if VL > 0"
 * (MCTSNode::update, src/mcts/mcts_node_virtual_loss.cpp:54-71) then the
 * clamped VL -= vl_value (revertVirtualLoss), node_visits[node] += 1, and
 * v = -v per ply (src/mcts/mcts_engine_batch_tree_simple.cpp:276-281).
 * Replaces launchBackupKernel (src/mcts/gpu_batch_evaluator.cpp:35-46).
 * The deepest edge receives +leaf_values[i], as the reference's loop adds
 * nn_output.value to the leaf node itself. */
int ob200_launch_backup(const ob200_tree_view* tree, const int32_t* paths,
                        const int32_t* path_len, const float* leaf_values, int32_t n,
                        int32_t max_depth, int32_t vl_value, ob200_stream stream);

/* P[node][slot] = clamp(policy[i][action_of_slot[node][slot]], 0, 1) for the
 * existing child slots of node_ids[i]; no renormalisation.
 * Replaces MCTSNode::setPriorProbabilities (src/mcts/mcts_node.cpp:512-593).
 * slot_action: [n_nodes][pitch] action id of each child slot, or NULL when
 * slot == action.  policy: [n][policy_size] fp32 on the device. */
int ob200_launch_set_priors(const ob200_tree_view* tree, const int32_t* node_ids, int32_t n,
                            const float* policy, int32_t policy_size,
                            const int32_t* slot_action, ob200_stream stream);

/* Root-to-leaf descent, one simulation after another inside each tree, trees
 * in parallel: sims_per_tree simulations from roots[t]; every step is the
 * selection above followed by VL += vl_value on the chosen edge, so that
 * simulation k sees the virtual loss of simulations < k of the same tree.
 * Descent stops at an edge whose child_node is -1 (leaf to expand) or after
 * max_depth steps.  (The simulations of a tree overlap as a wavefront, one
 * level apart; the result is that of running them one after another as long
 * as every node is reached at a single depth below its root, which holds for
 * trees and for games in which every move adds a stone.)  paths_out [n_trees*sims_per_tree][max_depth][2],
 * path_len_out [n_trees*sims_per_tree].
 * Replaces phase 1 of MCTSEngine::executeBatchedTreeSearch
 * (src/mcts/mcts_engine_batch_tree_simple.cpp:73-185) and
 * launchTreeTraversalKernel (include/mcts/gpu_kernels.h:9-26). */
int ob200_launch_traverse(const ob200_tree_view* tree, const int32_t* roots, int32_t n_trees,
                          int32_t sims_per_tree, float c_puct, int32_t vl_value,
                          int32_t max_depth, int32_t* paths_out, int32_t* path_len_out,
                          ob200_stream stream);

/* ------------------------------------------------------------------------- *
 *  Tree handle: the same operations with HOST buffers at the boundary, for a
 *  C++ search loop that keeps its own control flow and moves the per-node work
 *  of MCTSNode (include/mcts/mcts_node.h:39-101) to the device in batches - the
 *  calls MCTSEngine::executeBatchedTreeSearch makes one node at a time at
 *  src/mcts/mcts_engine_batch_tree_simple.cpp:100-111 (selectChild,
 *  applyVirtualLoss) and :249-281 (expand, setPriorProbabilities, update,
 *  revertVirtualLoss).  The handle owns the device arrays (ob200_tree_view_of
 *  gives them to the ob200_launch_* layer), its stream and page-locked staging;
 *  calls on one handle are serialised and return when their results are on the
 *  host.  Node ids are dense, in creation order.
 * ------------------------------------------------------------------------- */
typedef struct ob200_tree ob200_tree;
int ob200_tree_create(int32_t device, int32_t max_nodes, int32_t n_children, ob200_tree** out);
void ob200_tree_destroy(ob200_tree* tree);
/* Device arrays of the handle (n_nodes = capacity). */
int ob200_tree_view_of(ob200_tree* tree, ob200_tree_view* view_out);
int32_t ob200_tree_node_count(ob200_tree* tree);
/* Forgets every node (a new search). */
int ob200_tree_clear(ob200_tree* tree);
/* Appends n nodes with zero statistics and no child links; node i gets the child
 * slots whose bit is set in exists_bits[i * words_per_node ...] (words_per_node
 * >= ceil(n_children / 32)).  The slot set of a node is what MCTSNode::expand
 * (src/mcts/mcts_node.cpp:238-436) creates children for: the legal moves.
 * *first_id_out = id of the first new node.  OB200_ERR_TOO_LARGE beyond capacity. */
int ob200_tree_add_nodes(ob200_tree* tree, int32_t n, const uint32_t* exists_bits,
                         int32_t words_per_node, int32_t* first_id_out);
/* child_node[parent[i]][slot[i]] = child[i] (-1 unlinks): what expand's
 * children_ vector and updateChildReference (include/mcts/mcts_node.h) hold. */
int ob200_tree_link(ob200_tree* tree, int32_t n, const int32_t* parent, const int32_t* slot,
                    const int32_t* child);
/* ob200_launch_puct_select on HOST arrays: sel_out[i] for node_ids[i]. */
int ob200_tree_select(ob200_tree* tree, const int32_t* node_ids, int32_t n, float c_puct,
                      int32_t vl_value, int32_t apply_vl, int32_t* sel_out);
/* amount > 0: MCTSNode::addVirtualLoss(amount) on edge (node_ids[i], slots[i]);
 * amount < 0: removeVirtualLoss(-amount), clamped at zero; slots[i] < 0 skipped. */
int ob200_tree_virtual_loss(ob200_tree* tree, const int32_t* node_ids, const int32_t* slots,
                            int32_t n, int32_t amount);
/* ob200_launch_backup on HOST arrays. */
int ob200_tree_backup(ob200_tree* tree, const int32_t* paths, const int32_t* path_len,
                      const float* leaf_values, int32_t n, int32_t max_depth, int32_t vl_value);
/* ob200_launch_set_priors on HOST arrays (slot == action). */
int ob200_tree_set_priors(ob200_tree* tree, const int32_t* node_ids, int32_t n, const float* policy,
                          int32_t policy_size);
/* Rows [first_node, first_node + n_nodes) of one array to / from the host: N, W, P,
 * VL, CHILD rows of `pitch` 4-byte elements, EXISTS rows of `mask_words` words,
 * VISITS one int per node (pitch / mask_words as ob200_tree_view_of reports). */
enum { OB200_TREE_N = 0, OB200_TREE_W = 1, OB200_TREE_P = 2, OB200_TREE_VL = 3, OB200_TREE_CHILD = 4,
       OB200_TREE_EXISTS = 5, OB200_TREE_VISITS = 6 };
int ob200_tree_read(ob200_tree* tree, int32_t field, int32_t first_node, int32_t n_nodes, void* host_out);
int ob200_tree_write(ob200_tree* tree, int32_t field, int32_t first_node, int32_t n_nodes, const void* host_in);

/* ------------------------------------------------------------------------- *
 *  Board tensors: the activation format of the encoder and the network.
 *
 *  bf16, NHWC: element (channel c, board b, row y, column x) of a tensor with C
 *  channels lives at
 *        (G + b * slots + y * GP + x) * C + c
 *  with GP = board_size + 1 (one zero column after each row), slots = GP * GP
 *  (one zero row after each board), G = OB200_GUARD zero positions before the
 *  first and after the last board; the tensor has PT = 2 * G +
 *  roundup(B * slots, 128) positions.  The zero column / row / guards are the
 *  3x3 convolution's padding; every producer writes them as zero.  With C = 64
 *  one position is one 128-byte row, which is what the tensor-core kernel's
 *  TMA boxes and 128-byte-swizzled shared-memory tiles are built on.
 * ------------------------------------------------------------------------- */
#define OB200_GUARD 32
/* Storage type of a board tensor and of the packed tower weights.  BF16 is the
 * default everywhere.  F16 (same tensor-core rate, 11 significant bits instead
 * of 8, range up to 65,504 with activations saturating there instead of
 * overflowing) is for networks whose residual stream is not normalised, where 21
 * layers of bf16 rounding leave the logits several 1e-2 away from the fp32
 * forward of ResNetModel::forward (src/nn/resnet_model.cpp:104-237).  Every
 * tensor that meets in one call (input, weights, residual, output) must be of
 * the same type; calls without a dtype argument read and write bf16. */
#define OB200_DTYPE_BF16 0
#define OB200_DTYPE_F16 1
/* Positions (PT above) of a board tensor for a batch of B boards. */
int64_t ob200_board_tensor_positions(int32_t board_size, int32_t B);
/* Bytes of a board tensor with `channels` channels (rounded up to 8). */
int64_t ob200_board_tensor_bytes(int32_t board_size, int32_t B, int32_t channels);

/* Gomoku state -> input planes, written as a bf16 board tensor of
 * `out_channels` (a multiple of 8, >= planes) channels.
 * Replaces GomokuState::getEnhancedTensorRepresentation
 * (src/games/gomoku/gomoku_state.cpp:210-372), the attack/defense planes of
 * GomokuAttackDefenseModule::compute_planes (src/utils/attack_defense_module.cpp:61-111)
 * and the batching copy of ResNetModel::prepareInputTensor
 * (src/nn/resnet_model.cpp:240-576).
 *   history[b][k], k in [0, n_hist[b]) : the k-th most recent move (k = 0 is
 *       the last move played), action = row * board_size + col; n_hist <= 16.
 *   to_move[b] : 1 = BLACK, 2 = WHITE.
 *   planes : 17 or 19.  Plane 2i = the side to move's i-th most recent stone,
 *       plane 2i+1 = the opponent's i-th most recent stone (one stone per
 *       plane), plane 16 = all ones iff BLACK is to move, planes 17/18 = the
 *       attack / defense planes, which the reference's CPU code computes as
 *       zero for every legal move (it scores the board without the candidate
 *       stone against itself).
 * All pointers are device pointers; history must be 16-byte aligned (each
 * board's 16 entries are read as two 16-byte words). */
int ob200_launch_encode_gomoku(const int16_t* history, const uint8_t* n_hist,
                               const uint8_t* to_move, int32_t B, int32_t board_size,
                               int32_t planes, int32_t out_channels, void* board_tensor_out,
                               ob200_stream stream);
/* The same with the board tensor's storage type chosen (OB200_DTYPE_*). */
int ob200_launch_encode_gomoku_dt(const int16_t* history, const uint8_t* n_hist,
                                  const uint8_t* to_move, int32_t B, int32_t board_size,
                                  int32_t planes, int32_t out_channels, int32_t dtype,
                                  void* board_tensor_out, ob200_stream stream);

/* Gomoku board -> the reference's 3-plane representation, for networks built
 * with 3 input channels (src/nn/resnet_model.cpp:258-260).  Replaces
 * GomokuState::getTensorRepresentation (src/games/gomoku/gomoku_state.cpp:184-208):
 * channel 0 the stones of the side to move, 1 the opponent's, 2 all ones iff
 * BLACK is to move.  stones [B][S*S]: 0 empty, 1 black, 2 white; to_move [B]:
 * 1 BLACK, 2 WHITE; out_channels a multiple of 8.  Device pointers. */
int ob200_launch_encode_gomoku3(const int8_t* stones, const uint8_t* to_move, int32_t B,
                                int32_t board_size, int32_t out_channels, void* board_tensor_out,
                                ob200_stream stream);

/* The Gomoku attack / defense planes as an operator of its own.  Replaces
 * GomokuAttackDefenseModule::compute_planes / compute_bonuses
 * (src/utils/attack_defense_module.cpp:50-111, threat counts :205-222, :333-487).
 * stones [B][S*S] (0 empty, 1 black, 2 white), to_move [B]; attack_out,
 * defense_out [B][S*S] fp32, zero on occupied cells.  For an empty cell m:
 * attack = threats(after, mover) - threats(before, mover), defense =
 * threats(before, opponent) - threats(after, opponent), `before` with m empty.
 * stone_placed == 0 is compute_planes' call pattern: `after` is the position
 * itself, so both planes are zero everywhere (what the encoders write into
 * planes 17 / 18).  stone_placed != 0: `after` has the mover's stone on m, as
 * compute_bonuses is called with a board that already holds the chosen move.
 * Device pointers; board_size in [6, 32]. */
int ob200_launch_gomoku_attack_defense(const int8_t* stones, const uint8_t* to_move, int32_t B,
                                       int32_t board_size, int32_t stone_placed, float* attack_out,
                                       float* defense_out, ob200_stream stream);

/* Chess state -> the reference's 20 input planes, written as a bf16 board
 * tensor (board_size 8) of `out_channels` (a multiple of 8, >= 24) channels.
 * Replaces ChessState::getEnhancedTensorRepresentation
 * (src/games/chess/chess_state.cpp:745-826) with the CPU code of
 * computeAttackDefensePlanes (:1753-1803).  Square = rank * 8 + file.
 *   pieces [B][64] : 0 empty, else 1..6 = pawn, knight, bishop, rook, queen,
 *       king, + 8 for black;
 *   meta [B][6] : side to move (1 white, 2 black), castling bits (1 WK, 2 WQ,
 *       4 BK, 8 BQ), en passant square or -1, halfmove clock, chess960 (0/1),
 *       how often the position has occurred (the repetition plane is that / 3);
 *   legal_to [B][2] : 64-bit set of the destination squares of the legal moves
 *       (move generation stays with the caller).
 * Planes: 0-5 white P N B R Q K, 6-11 black, 12 side to move, 13 castling,
 * 14 en passant, 15 halfmove / 100, 16 chess960, 17 repetition, 18 / 19 value
 * of enemy / own pieces around each legal destination.  Values are the
 * reference's fp32 values rounded to bf16.  All pointers are device pointers. */
int ob200_launch_encode_chess(const int8_t* pieces, const int32_t* meta, const uint32_t* legal_to,
                              int32_t B, int32_t out_channels, void* board_tensor_out,
                              ob200_stream stream);

/* Go state -> the reference's 10 input planes, written as a bf16 board tensor of
 * `out_channels` (a multiple of 8, >= 10) channels.  Replaces
 * GoState::getEnhancedTensorRepresentation (src/games/go/go_state.cpp:596-704)
 * with the CPU code of computeAttackDefensePlanes (:1306-1476): planes 0 / 1
 * black / white stones, 2 all ones iff black is to move, 3 / 4 min(1, liberties /
 * 10) of the black / white group on its stones, 5 ko point, 6 / 7 distance to
 * the nearer edge over S/2, 8 / 9 capture / liberty-defense scores of the legal
 * cells.  Values are the reference's fp32 values rounded to bf16.
 *   stones [B][S*S] : 0 empty, 1 black, 2 white;  ko_point [B] : cell or -1;
 *   to_move [B] : 1 black, 2 white;  legal_bits [B][ceil(S*S/32)] : bit p set
 *   iff cell p is in GoState::getLegalMoves() (the rules - suicide, ko,
 *   superko - stay with the caller, which needs the legal moves anyway).
 * All pointers are device pointers.  board_size <= 30. */
int ob200_launch_encode_go(const int8_t* stones, const int32_t* ko_point, const uint8_t* to_move,
                           const uint32_t* legal_bits, int32_t B, int32_t board_size,
                           int32_t out_channels, void* board_tensor_out, ob200_stream stream);

/* fp32 planes [B][C][S][S] (NCHW, device) -> bf16 board tensor of out_channels
 * channels; channels >= C are zero.  The reference feeds such planes from
 * IGameState::getTensorRepresentation / getEnhancedTensorRepresentation
 * (include/core/igamestate.h:141,151) through prepareInputTensor. */
int ob200_launch_planes_to_board_tensor(const float* planes_nchw, int32_t B, int32_t C,
                                        int32_t board_size, int32_t out_channels,
                                        void* board_tensor_out, ob200_stream stream);
/* The same with the board tensor's storage type chosen (OB200_DTYPE_*); fp16 rounds
 * to nearest even and magnitudes beyond 65,504 become infinity, as a conversion of
 * the planes to torch.float16 would. */
int ob200_launch_planes_to_board_tensor_dt(const float* planes_nchw, int32_t B, int32_t C,
                                           int32_t board_size, int32_t out_channels, int32_t dtype,
                                           void* board_tensor_out, ob200_stream stream);

/* One 3x3 convolution layer (padding 1, stride 1) on board tensors with the
 * BatchNorm already folded into weight and bias:
 *   out = act(conv3x3(in, w) + bias [+ residual]),  act = ReLU if relu != 0.
 * Replaces one conv + BatchNorm2d + relu (+ residual add) group of
 * ResNetResidualBlock::forward / ResNetModel::forward
 * (src/nn/resnet_model.cpp:43-49,150).  `packed_w` comes from
 * ob200_pack_conv3x3_weights.  in, out and residual are 64-channel board
 * tensors of B boards (cin = cout = 64 in this build; a layer with fewer real
 * input channels, like the stem, runs with zero weights on the rest). */
int ob200_launch_conv3x3(const void* in, const void* packed_w, const float* bias,
                         const void* residual, void* out, int32_t B, int32_t board_size,
                         int32_t cin, int32_t cout, int32_t relu, ob200_stream stream);
/* The same on tensors and packed weights of storage type `dtype` (OB200_DTYPE_*).
 * fp16 outputs saturate at +-65,504 instead of overflowing to infinity. */
int ob200_launch_conv3x3_dt(const void* in, const void* packed_w, const float* bias,
                            const void* residual, void* out, int32_t B, int32_t board_size,
                            int32_t cin, int32_t cout, int32_t relu, int32_t dtype,
                            ob200_stream stream);
/* Bytes of the packed bf16 weight image for (cin, cout); 0 when unsupported. */
int64_t ob200_packed_conv3x3_bytes(int32_t cin, int32_t cout);
/* Host helper: fp32 OIHW weights [cout][cin_real][3][3] scaled per output
 * channel by scale[cout] (the folded BatchNorm factor; NULL = 1) -> packed
 * bf16 image for cin >= cin_real input channels (extra channels get zero
 * weights).  Output is HOST memory of ob200_packed_conv3x3_bytes(cin, cout);
 * copy it to the device for ob200_launch_conv3x3. */
int ob200_pack_conv3x3_weights(const float* w_oihw, const float* scale, int32_t cout,
                               int32_t cin_real, int32_t cin, void* packed_out);
/* The same, rounding to `dtype` (OB200_DTYPE_*); the image has the same size. */
int ob200_pack_conv3x3_weights_dt(const float* w_oihw, const float* scale, int32_t cout,
                                  int32_t cin_real, int32_t cin, int32_t dtype, void* packed_out);

/* ------------------------------------------------------------------------- *
 *  Network handle: the residual policy/value network.
 *  Replaces alphazero::nn::ResNetModel behind NeuralNetwork::inference
 *  (include/nn/neural_network.h:28-29, src/nn/resnet_model.cpp:51-237,594-811).
 * ------------------------------------------------------------------------- */
typedef struct ob200_net ob200_net;

typedef struct ob200_net_config {
    int32_t board_size;       /* S: 15 for Gomoku                              */
    int32_t input_channels;   /* C_in of the stem (17, 19, 3, ...)             */
    int32_t filters;          /* tower width: 64, 128 or 256                   */
    int32_t blocks;           /* residual blocks                               */
    int32_t policy_size;      /* A: policy outputs                             */
    int32_t policy_head_ch;   /* channels of the policy 1x1 conv (reference 32)*/
    int32_t value_head_ch;    /* channels of the value 1x1 conv (reference 32) */
    int32_t value_hidden;     /* width of value_fc1 (reference 256)            */
    int32_t max_batch;        /* largest batch any call will pass              */
    int32_t device;           /* CUDA device ordinal                           */
    int32_t policy_kind;      /* OB200_POLICY_FC (the reference's head) or
                                 OB200_POLICY_CONV_PLANES                       */
    int32_t tower_dtype;      /* OB200_DTYPE_BF16 (0) or OB200_DTYPE_F16: storage
                                 type of the tower's weights and of every board
                                 tensor of this handle, the input tensor of
                                 ob200_net_forward_device included.  The heads
                                 compute in fp32 either way.                    */
} ob200_net_config;

/* Policy head kinds.  FC: 1x1 conv to policy_head_ch channels + BatchNorm + ReLU
 * + policy_fc, as ResNetModel (src/nn/resnet_model.cpp:81-88,:178-188).
 * CONV_PLANES (no counterpart in the reference; the shape of the chess
 * configuration): 1x1 convolution with bias to policy_head_ch planes, logits =
 * the planes flattened in NCHW order (index = plane * S^2 + cell), policy_size
 * = policy_head_ch * S^2; tensors "policy_conv.weight" [planes][filters][1][1]
 * and "policy_conv.bias" [planes]; filters 128 or 256 only. */
#define OB200_POLICY_FC 0
#define OB200_POLICY_CONV_PLANES 1

int ob200_net_create(const ob200_net_config* cfg, ob200_net** out);
void ob200_net_destroy(ob200_net* net);

/* Weights enter under the reference module's parameter / buffer names
 * (src/nn/resnet_model.cpp:51-102): "input_conv.weight",
 * "input_bn.{weight,bias,running_mean,running_var}",
 * "res_blocks.<i>.{conv1,bn1,conv2,bn2}.*", "policy_conv.weight", "policy_bn.*",
 * "policy_fc.{weight,bias}", "value_conv.weight", "value_bn.*",
 * "value_fc1.{weight,bias}", "value_fc2.{weight,bias}"; fp32, the layout
 * libtorch stores (OIHW / [out][in]).  "*.num_batches_tracked" is accepted and
 * ignored.  Replaces ResNetModel::load (src/nn/resnet_model.cpp:836-857) at
 * the level of tensors. */
int ob200_net_set_tensor(ob200_net* net, const char* name, const float* data, int64_t numel);
/* Folds BatchNorm (eps 1e-5) into the convolutions, rounds tower weights to
 * bf16, permutes what needs permuting and uploads.  Fails with OB200_ERR_STATE
 * naming the first tensor that was never set. */
int ob200_net_finalize(ob200_net* net);

#define OB200_OUT_PROBS 0   /* policy_out = softmax probabilities (what
                               ResNetModel::inference returns, :752)          */
#define OB200_OUT_LOGITS 1  /* policy_out = policy_fc outputs before softmax  */

/* HOST in, HOST out.  planes: fp32 [B][C][S][S]; as ResNetModel::forward does
 * (src/nn/resnet_model.cpp:117-147) the first min(C, input_channels) planes
 * are used and missing ones are zero.  policy_out [B][A], value_out [B]. */
int ob200_net_infer_planes(ob200_net* net, const float* planes, int32_t B, int32_t C,
                           float* policy_out, float* value_out, int32_t out_kind);
/* HOST in, HOST out, Gomoku states given as move histories (see
 * ob200_launch_encode_gomoku): encode -> tower -> heads in one call.  This is
 * the call behind NeuralNetwork::inference for Gomoku states. */
int ob200_net_infer_gomoku(ob200_net* net, const int16_t* history, const uint8_t* n_hist,
                           const uint8_t* to_move, int32_t B, float* policy_out,
                           float* value_out, int32_t out_kind);
/* The same call split in two, so that one thread can keep two batches in flight:
 * submit returns when the work is enqueued (*ticket_out names the call), wait
 * returns when its results are in policy_out / value_out.  While the results of
 * one batch travel back to the host the kernels of the next one run.  At most two
 * calls may be pending per handle (a third submit returns OB200_ERR_STATE); all
 * buffers of a call must stay valid and untouched until its wait returns; every
 * submitted ticket must be waited for before the handle is destroyed.  (The
 * one-call forms above overlap in the same way when several threads call them
 * on one handle, which is how the reference's engines call NeuralNetwork::inference
 * when no global queue is set, src/mcts/mcts_engine_batch_tree_simple.cpp:231-233.) */
int ob200_net_submit_gomoku(ob200_net* net, const int16_t* history, const uint8_t* n_hist,
                            const uint8_t* to_move, int32_t B, float* policy_out,
                            float* value_out, int32_t out_kind, int32_t* ticket_out);
int ob200_net_wait(ob200_net* net, int32_t ticket);
/* DEVICE in, DEVICE out, asynchronous on `stream`: input is a board tensor of
 * ob200_net_input_tensor_channels() channels holding B <= max_batch boards
 * (ob200_board_tensor_bytes(board_size, B, channels) bytes, 16-byte aligned). */
int ob200_net_forward_device(ob200_net* net, const void* input_board_tensor, int32_t B,
                             float* policy_out, float* value_out, int32_t out_kind,
                             ob200_stream stream);
/* DEVICE in, DEVICE out, asynchronous on `stream`, Gomoku positions given as move
 * histories (the arrays of ob200_launch_encode_gomoku, history 16-byte aligned):
 * encode -> tower -> heads.  On the board-resident tower path (64 filters, boards
 * up to 15x15) the tower kernel writes its own input planes from the histories -
 * no encoder launch and no input tensor in device memory; on the other paths the
 * encoder kernel runs first.  Results are those of ob200_launch_encode_gomoku +
 * ob200_net_forward_device. */
int ob200_net_forward_gomoku_device(ob200_net* net, const int16_t* history, const uint8_t* n_hist,
                                    const uint8_t* to_move, int32_t B, float* policy_out,
                                    float* value_out, int32_t out_kind, ob200_stream stream);
/* Device pointer of the tower's output board tensor of the last forward
 * (filters channels), for tests. */
const void* ob200_net_debug_tower_output(ob200_net* net);
/* Which tower path the last forward took, for tests and measurements:
 * 0 one launch per layer, 1 one cooperative launch (tiles handed over through
 * flags), 2 one launch with the boards resident in shared memory; -1 before the
 * first forward.  Environment, read when a handle is finalised:
 * OB200_TOWER_RESIDENT=0 switches path 2 off; OB200_TOWER_FUSED=0 / 2 switches
 * path 1 off / forces it at every batch size (and, unless OB200_TOWER_RESIDENT=1,
 * switches path 2 off). */
int32_t ob200_net_debug_tower_path(ob200_net* net);
/* The residual tower alone (stem + blocks), DEVICE in, asynchronous on `stream`;
 * the result is the board tensor ob200_net_debug_tower_output() points at.
 * For measurement and for callers that run their own heads. */
int ob200_net_tower_device(ob200_net* net, const void* input_board_tensor, int32_t B,
                           ob200_stream stream);
/* The value head alone, for callers that must never allocate.  (No counterpart in
 * the reference: its value head runs inside ResNetModel::forward on libtorch's
 * caching allocator.)  Meant for search threads in the middle of a self-play loop
 * and for processes whose device memory is budgeted once at start-up: a cudaMalloc
 * there synchronises the whole device and stalls every other engine's stream, or
 * simply fails when the budget is spent.  This call allocates nothing, on the
 * device or the host: the two intermediates of the value head (1x1-convolution
 * activations and the hidden layer) live in one array compiled into the library,
 * 2 MiB per GPU, held by every GPU that loads the library until the process ends.
 *   tower_board_tensor : DEVICE, 64-channel board tensor of B boards (the tower's
 *       output, e.g. ob200_net_debug_tower_output after a forward);
 *   value_out : DEVICE, B floats, tanh values; weights come from the handle.
 * Limit: B * (value_head_ch * S * S + value_hidden) <= the capacity below (in
 * floats; 524,288 = batch 1089 for the 15x15, 1-channel head); more returns
 * OB200_ERR_TOO_LARGE.  The first call on each device looks the array's address up;
 * make that first call outside any stream capture.  All calls on a device share the
 * array, which keeps whatever the last call left: nothing needs clearing because each
 * launch overwrites what the next one reads, but two calls whose kernels overlap on
 * the GPU (different streams, no ordering) race on it — order them.  Asynchronous on
 * `stream`; results are identical to the value output of ob200_net_forward_device. */
int ob200_net_value_head_noalloc(ob200_net* net, const void* tower_board_tensor, int32_t B,
                                 float* value_out, ob200_stream stream);
int64_t ob200_value_head_noalloc_capacity(void);

/* Channel count of the input board tensor ob200_net_forward_device expects
 * (64: the stem runs on the same 64-channel kernel as the tower, with zero
 * weights for the channels beyond input_channels). */
int32_t ob200_net_input_tensor_channels(ob200_net* net);

/* Reads and clears the current device's error word, which a kernel raises when
 * one of its bounded waits (on a copy or a tensor-core completion barrier)
 * runs out: 0 = none.  Synchronises the device.  The host-buffer calls above
 * check it themselves and return OB200_ERR_TIMEOUT. */
int ob200_device_error_code(int32_t* code_out);
/* Test hook for that path: one thread waits on a barrier nobody arrives at,
 * gives up after spin_limit polls (microseconds) and raises the error word with
 * code 9.  Nothing faults or hangs; the context stays usable. */
int ob200_debug_bounded_wait(int32_t spin_limit, ob200_stream stream);

/* ------------------------------------------------------------------------- *
 *  Leaf-parallel search, Gomoku, device-resident trees.
 *  Replaces MCTSEngine::runSearch / executeBatchedTreeSearch
 *  (src/mcts/mcts_engine_search.cpp:347-406,
 *  src/mcts/mcts_engine_batch_tree_simple.cpp:14-301) for a group of
 *  independent games on one GPU, together with MCTSNode::expand
 *  (src/mcts/mcts_node.cpp:238-436), addDirichletNoise
 *  (src/mcts/mcts_engine_eval.cpp:83-110) and getActionProbabilities
 *  (src/mcts/mcts_engine_tree.cpp:389-465).
 *
 *  Per move and per tree: the root is created from the game's move list and
 *  evaluated once (priors = network policy, optionally mixed with Dirichlet
 *  noise); then rounds of { descend leaf_batch / n_trees simulations per tree
 *  with virtual loss (ob200_launch_traverse), rebuild each leaf's position from
 *  the path, detect five-in-a-row / full board, encode, network forward, expand
 *  (one new node per leaf edge, priors = clamp(policy), no renormalisation),
 *  back up with virtual-loss revert } until sims_per_move simulations per tree
 *  are done.  No host synchronisation inside a move.
 *  Where the reference leaves things open or racy this defines them:
 *  children are in action order (the reference shuffles them); simulations of a
 *  tree inside a round run in sequence; a leaf reached twice in a round is
 *  expanded once (by the simulation with the lowest index; nodes are numbered in
 *  simulation order, so a search is reproducible bit for bit) and backed up twice; a terminal leaf takes the game result
 *  (-1 for the side to move after a five-in-a-row, 0 for a full board) instead
 *  of the network value (the reference's batched loop asks the network even
 *  then; its serial loop uses the result); value_sign = +1 adds the leaf value
 *  to the leaf edge as the reference's batched loop does, -1 is negamax.
 *  Transposition table (replaces PHMapTranspositionTable,
 *  src/mcts/phmap_transposition_table.cpp, as the batched loop uses it,
 *  mcts_engine_batch_tree_simple.cpp:117-162): when a leaf edge is expanded and
 *  a node with the same Zobrist key (stones + side to move, as
 *  GomokuState::compute_hash_signature_internal) already exists in this move's
 *  trees, the edge is pointed at
 *  that node instead of a new one, so the subtree and its statistics are shared.
 * ------------------------------------------------------------------------- */
typedef struct ob200_search ob200_search;

enum { OB200_RULES_FREESTYLE = 0, OB200_RULES_OMOK = 1, OB200_RULES_RENJU = 2 };

typedef struct ob200_search_config {
    int32_t n_trees;            /* concurrent games on this GPU                    */
    int32_t sims_per_move;      /* simulations per tree per move (800)             */
    int32_t leaf_batch;         /* leaves per network call, multiple of n_trees    */
    int32_t max_depth;          /* longest path recorded (<= 64)                   */
    float c_puct;               /* MCTSSettings::exploration_constant              */
    int32_t virtual_loss;       /* MCTSSettings::virtual_loss (3)                  */
    float dirichlet_alpha;      /* 0.3                                             */
    float dirichlet_epsilon;    /* 0.25; 0 disables the root noise                 */
    int32_t value_sign;         /* +1 reference batched loop, -1 negamax           */
    int32_t use_transposition_table; /* MCTSSettings::use_transposition_table      */
    uint64_t seed;              /* root-noise generator, Zobrist keys, widening    */
    /* MCTSNode::expand's two limits on the children a node gets
     * (src/mcts/mcts_node.cpp:283-340).  max_children: the first max_children
     * legal moves in move order; 0 = the reference's 1,000 (never reached on a
     * 225-move board).  use_progressive_widening (MCTSSettings, off in the shipped
     * configuration): a node keeps a random subset of
     * max(8, progressive_widening_c * (visits + 1)^progressive_widening_k) of its
     * legal moves; a node is expanded once, with no visits yet, so the count is
     * max(8, floor(c)).  The subset is a function of (seed, number of
     * ob200_search_run calls so far, node id). */
    int32_t max_children;
    int32_t use_progressive_widening;
    float progressive_widening_c;
    float progressive_widening_k;
    /* The Gomoku variant (GomokuState's use_renju / use_omok constructor flags,
     * src/games/gomoku/gomoku_state.cpp:23-31, :915-943): OB200_RULES_*.  Omok
     * denies BLACK a move that makes six or more in a row or open threes in two
     * directions (src/games/gomoku/gomoku_rules.cpp:118-198); a win is five or more
     * for either side, as in freestyle.  Renju denies BLACK overlines, double
     * fours and double threes as the reference defines them (:200-879; an exact
     * five is always allowed), and BLACK wins only with exactly five and no longer
     * line through the stone (gomoku_state.cpp:812-843).  The double-three test
     * follows the cell that would complete a three through at most four nested
     * levels.  The opening restriction (use_pro_long_opening) is not built. */
    int32_t rules;
} ob200_search_config;

typedef struct ob200_search_stats {
    int64_t simulations;        /* all trees, this call                            */
    int64_t evaluations;        /* positions sent to the network (roots included)  */
    int64_t nodes;              /* nodes allocated, all trees                      */
    int64_t terminal_leaves;    /* simulations that ended in a finished game       */
    double device_ms;           /* device time of the enqueued work (CUDA events)  */
    double wall_ms;             /* host time of the whole call: root set-up, noise
                                   sampling, copies, the wait and the read-back
                                   included                                        */
} ob200_search_stats;

/* `net` must be a finalised 15x15 Gomoku network with max_batch >= leaf_batch;
 * the search borrows it (destroy the search first). */
int ob200_search_create(ob200_net* net, const ob200_search_config* cfg, ob200_search** out);
void ob200_search_destroy(ob200_search* s);
/* One move for every tree.  HOST buffers.  moves[t * moves_stride + i], i in
 * [0, n_moves[t]): the game so far (BLACK first), legal and unfinished.
 * pi_out [n_trees][225]: visit counts -> (n / n_max)^(1/T) normalised, one-hot
 * argmax for temperature < 0.01; visits_out [n_trees][225] may be NULL. */
int ob200_search_run(ob200_search* s, const int16_t* moves, const int32_t* n_moves, int32_t moves_stride,
                     float temperature, float* pi_out, int32_t* visits_out, ob200_search_stats* stats);
/* Test hooks: device pointers of the search's tree view and node counter, and a
 * synchronous device-to-host copy for reading them. */
int ob200_search_debug_tree(ob200_search* s, ob200_tree_view* view_out, int32_t* nodes_used_out);
/* More test hooks, for comparing a search with a CPU restatement fed the same
 * network outputs.  value_quantum > 0: network values are rounded to multiples
 * of 1 / value_quantum before they are backed up (sums of such values are exact
 * in fp32 whatever the order of the atomic additions).  record_rounds > 0: the
 * policy [leaf_batch][225] and value [leaf_batch] arrays of the root evaluation
 * (entry 0, n_trees rows used) and of the first record_rounds rounds of every
 * later ob200_search_run are kept on the device; ob200_search_debug_record gives
 * their device pointers ([record_rounds + 1] entries each) and the root noise
 * [n_trees][228] of the last run. */
int ob200_search_debug_hooks(ob200_search* s, float value_quantum, int32_t record_rounds);
int ob200_search_debug_record(ob200_search* s, const float** policy_out, const float** value_out,
                              const float** noise_out);
/* Measurement hook.  enable != 0: the next ob200_search_run calls record events
 * around the five phases of every round (descent, leaf positions, network,
 * expansion, backup); the events break the programmatic-dependent chain between
 * the phases, so such a run is a little slower than a plain one.  phase_ms_out
 * (5 doubles, may be NULL) receives the sums over the rounds of the last run
 * that was timed this way. */
int ob200_search_debug_phases(ob200_search* s, int32_t enable, double* phase_ms_out);
int ob200_copy_to_host(void* dst_host, const void* src_device, int64_t bytes);

/* Per-device counters for the end-of-run reduction (the only cross-GPU step;
 * it replaces the MCTSStats fields total_evaluations / total_batches_processed,
 * include/mcts/mcts_engine.h:154-197). */
typedef struct ob200_counters {
    uint64_t evals;            /* positions evaluated by the network          */
    uint64_t batches;          /* network calls                               */
    uint64_t selections;       /* node selections made                        */
    uint64_t backups;          /* paths backed up                             */
    uint64_t kernel_launches;  /* kernels of this library launched            */
} ob200_counters;
int ob200_get_counters(ob200_counters* out);   /* this process, all handles   */
void ob200_reset_counters(void);

#ifdef __cplusplus
}
#endif
#endif /* OMOKNUNI_B200_H */
