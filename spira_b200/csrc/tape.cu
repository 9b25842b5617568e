// spira_b200_run_tape: the operators of a recorded network forward, executed in order by one call into the library.
//
// The executor owns no memory and keeps no state between calls: feature tensors that only live inside the forward pass
// are placed in the caller's arena (slots with the same buffer number share storage; the caller derives the numbers from
// the lifetimes of the recorded pass), the kernel maps of the scene come in as a table of pointers, and every operator
// is resolved to one spira_b200_conv descriptor or one spira_b200_pointwise call.
#include "common.cuh"

#include <vector>

using namespace sb;

namespace {

constexpr size_t kArenaAlign = 256;

// the Python binding mirrors these layouts field by field
static_assert(sizeof(spira_b200_conv_desc) == 192, "spira_b200_conv_desc layout");
static_assert(sizeof(spira_b200_tape_map) == 128, "spira_b200_tape_map layout");
static_assert(sizeof(spira_b200_tape_op) == 112, "spira_b200_tape_op layout");
static_assert(sizeof(spira_b200_tape_slot) == 24, "spira_b200_tape_slot layout");

inline size_t round_up(size_t n, size_t a) { return (n + a - 1) / a * a; }

}  // namespace

extern "C" int spira_b200_run_tape(const spira_b200_tape_op *ops, int n_ops, const spira_b200_tape_map *maps, int n_maps,
                                   spira_b200_tape_slot *slots, int n_slots, void *arena, size_t arena_bytes,
                                   size_t *arena_needed, float *zeroed_accum, size_t zeroed_accum_floats, int32_t *status,
                                   void *stream) {
  SB_CHECK_ARG(n_ops >= 0 && n_maps >= 0 && n_slots >= 0 && (ops || n_ops == 0) && (maps || n_maps == 0) && (slots || n_slots == 0),
               "run_tape: null table");
  // ---- place the slots that live in the arena: one region per buffer number, as large as its largest slot
  int n_buffers = 0;
  for (int s = 0; s < n_slots; ++s) {
    SB_CHECK_ARG(slots[s].rows >= 0 && slots[s].channels >= 0, "run_tape: slot %d has rows=%lld channels=%d", s,
                 static_cast<long long>(slots[s].rows), slots[s].channels);
    SB_CHECK_ARG(slots[s].buffer >= -1, "run_tape: slot %d has buffer %d", s, slots[s].buffer);
    if (slots[s].buffer >= n_buffers) n_buffers = slots[s].buffer + 1;
  }
  std::vector<size_t> size(static_cast<size_t>(n_buffers), 0), offset(static_cast<size_t>(n_buffers), 0);
  for (int s = 0; s < n_slots; ++s) {
    if (slots[s].ptr != nullptr || slots[s].buffer < 0) continue;
    const size_t bytes = static_cast<size_t>(slots[s].rows) * slots[s].channels * sizeof(__half);
    if (bytes > size[slots[s].buffer]) size[slots[s].buffer] = bytes;
  }
  size_t total = 0;
  for (int b = 0; b < n_buffers; ++b) {
    offset[b] = total;
    total += round_up(size[b], kArenaAlign);
  }
  if (arena_needed) *arena_needed = total;
  if (total > arena_bytes || (total > 0 && arena == nullptr))
    return fail(SPIRA_B200_ERR_UNSUPPORTED, "run_tape: the arena holds %zu bytes, this scene needs %zu", arena_bytes, total);
  SB_CHECK_ARG(total == 0 || reinterpret_cast<uintptr_t>(arena) % kArenaAlign == 0, "run_tape: the arena must be 256-byte aligned");
  for (int s = 0; s < n_slots; ++s)      // (a slot with neither an address nor a buffer must not be named by an operator)
    if (slots[s].ptr == nullptr && slots[s].buffer >= 0) slots[s].ptr = static_cast<unsigned char *>(arena) + offset[slots[s].buffer];

  // ---- the operators
  auto slot_ok = [&](int s) { return s >= 0 && s < n_slots; };
  for (int i = 0; i < n_ops; ++i) {
    const spira_b200_tape_op &op = ops[i];
    SB_CHECK_ARG(slot_ok(op.in_a) && slot_ok(op.out) && (op.in_b == -1 || slot_ok(op.in_b)) && (op.residual == -1 || slot_ok(op.residual)),
                 "run_tape: operator %d names a slot outside [0, %d)", i, n_slots);
    const spira_b200_tape_slot &in_a = slots[op.in_a], &out = slots[op.out];
    SB_CHECK_ARG((in_a.ptr || in_a.rows == 0) && (out.ptr || out.rows == 0) && (op.in_b < 0 || slots[op.in_b].ptr || slots[op.in_b].rows == 0) &&
                     (op.residual < 0 || slots[op.residual].ptr || out.rows == 0),
                 "run_tape: operator %d uses a slot that has neither an address nor an arena buffer", i);
    SB_CHECK_ARG(out.channels == op.c_out, "run_tape: operator %d writes %d channels into a slot of %d", i, op.c_out, out.channels);
    const int c_a = op.in_b >= 0 ? op.c_in_a : op.c_in;
    SB_CHECK_ARG(in_a.channels == c_a && (op.in_b < 0 || slots[op.in_b].channels == op.c_in - c_a),
                 "run_tape: operator %d reads %d (+%d) channels, its slots hold %d (+%d)", i, c_a, op.c_in - c_a, in_a.channels,
                 op.in_b >= 0 ? slots[op.in_b].channels : 0);
    spira_b200_epilogue ep = op.epilogue;
    ep.residual = nullptr;
    if (op.residual >= 0) {
      SB_CHECK_ARG(slots[op.residual].rows == out.rows && slots[op.residual].channels == op.c_out,
                   "run_tape: operator %d: the residual slot does not match the output", i);
      ep.residual = slots[op.residual].ptr;
    }
    if (op.kind == SPIRA_B200_TAPE_POINTWISE) {
      SB_CHECK_ARG(op.in_b < 0 && op.residual < 0 && in_a.rows == out.rows, "run_tape: operator %d: a pointwise layer has one input and no residual", i);
      int rc = spira_b200_pointwise(in_a.ptr, op.weights, ep.bias, out.rows, op.c_in, op.c_out, out.ptr, stream);
      if (rc != SPIRA_B200_OK) return rc;
      continue;
    }
    spira_b200_conv_desc d{};
    d.K = op.K; d.c_in = op.c_in; d.c_out = op.c_out;
    d.c_in_a = c_a;
    d.feats = in_a.ptr;
    d.feats_b = op.in_b >= 0 ? slots[op.in_b].ptr : nullptr;
    d.packed = op.packed;
    d.weights = op.weights;
    d.epilogue = &ep;
    d.out = out.ptr;
    if (op.kind == SPIRA_B200_TAPE_IDENTITY) {
      SB_CHECK_ARG(op.K == 1 && in_a.rows == out.rows && (op.in_b < 0 || slots[op.in_b].rows == out.rows),
                   "run_tape: operator %d: a 1x1x1 layer keeps the rows of its input", i);
      d.dataflow = 0;
      d.num_sources = d.num_targets = out.rows;
    } else {
      SB_CHECK_ARG(op.kind == SPIRA_B200_TAPE_CONV, "run_tape: operator %d has unknown kind %d", i, op.kind);
      SB_CHECK_ARG(op.map >= 0 && op.map < n_maps, "run_tape: operator %d names map %d of %d", i, op.map, n_maps);
      const spira_b200_tape_map &m = maps[op.map];
      d.dataflow = op.dataflow;
      d.num_sources = op.transposed ? m.num_targets : m.num_sources;
      d.num_targets = op.transposed ? m.num_sources : m.num_targets;
      SB_CHECK_ARG(in_a.rows == d.num_sources && out.rows == d.num_targets && (op.in_b < 0 || slots[op.in_b].rows == d.num_sources),
                   "run_tape: operator %d: slots of %lld -> %lld rows on a map of %lld -> %lld", i, static_cast<long long>(in_a.rows),
                   static_cast<long long>(out.rows), static_cast<long long>(d.num_sources), static_cast<long long>(d.num_targets));
      if (op.dataflow == 0) {
        const int32_t *grouped = op.transposed ? m.grouped_map_t : m.grouped_map;
        if (op.grouped && grouped != nullptr) {
          d.map_os = grouped;
          d.row_of = op.transposed ? m.row_of_t : m.row_of;
          d.tile_masks = op.transposed ? m.tile_masks_t : m.tile_masks;
        } else {
          d.map_os = op.transposed ? m.map_os_t : m.map_os;
        }
        SB_CHECK_ARG(d.map_os != nullptr, "run_tape: operator %d runs output-stationary but map %d has no such form", i, op.map);
      } else {
        SB_CHECK_ARG(m.naddrs != nullptr, "run_tape: operator %d runs weight-stationary but map %d has no pair lists", i, op.map);
        SB_CHECK_ARG(static_cast<size_t>(d.num_targets) * op.c_out <= zeroed_accum_floats && zeroed_accum != nullptr,
                     "run_tape: operator %d needs %lld floats of zero scratch, %zu given", i,
                     static_cast<long long>(d.num_targets) * op.c_out, zeroed_accum_floats);
        d.in_idx = m.in_idx; d.out_idx = m.out_idx; d.naddrs = m.naddrs; d.qnaddrs = m.qnaddrs;
        d.rows = m.rows;
        d.mirror = m.mirror;
        d.swap = op.transposed ? 1 : 0;
        d.num_tiles128 = m.num_tiles128;
        d.zeroed_accum = zeroed_accum;
      }
    }
    int rc = conv_run(d, status, stream);
    if (rc != SPIRA_B200_OK) return rc;
  }
  return SPIRA_B200_OK;
}
