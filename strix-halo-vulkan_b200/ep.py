"""Host-side statement of the expert-parallel plan the device kernels follow (csrc/ep.cuh): which rank owns
an expert, where a rank's rows sit in the gathered order, which (row, expert) pairs a rank computes and
where each pair's output goes. The reference keeps every expert on one device
(llm/gpu_moe.go:693-705), so there is no reference code for this; what must hold is that the exchange
changes no arithmetic: the row's owner adds its pairs in slot order, then the shared expert
(llm/moe.go:347-357, 403-406), exactly as a single device does.

Used by the multi-rank launcher (`connect`) and by the CPU tests, which run the plan over gloo ranks and
compare it with the single-rank result.
"""
import numpy as np


def expert_range(rank, world, n_expert):
    """Experts [lo, hi) that `rank` owns: contiguous, equal shares."""
    if n_expert % world:
        raise ValueError("the expert count must divide evenly over the ranks")
    per = n_expert // world
    return rank * per, (rank + 1) * per


def gathered_row(rank, rows, i):
    """Global index of rank's local row i when every rank contributes `rows` rows."""
    return rank * rows + i


def work_list(topk_g, rank, world, n_expert, entry_cols=8):
    """The work list rank `rank` builds from the gathered routing topk_g [world * rows][used] (the device's
    build_work_list with an expert filter): entries (expert or -1 for the shared expert, first column, columns)
    of at most entry_cols columns, and cols, the pair ids in expert-sorted order. Pair id = global row *
    (used + 1) + slot; slot == used is the shared expert, which a rank runs for its own rows only. The order of
    the pairs inside one expert is not specified (the device fills them with atomics); a pair's result does
    not depend on it."""
    topk_g = np.asarray(topk_g)
    rows_all, used = topk_g.shape
    rows = rows_all // world
    lo, hi = expert_range(rank, world, n_expert)
    entries, cols = [], []
    for e in range(lo, hi):
        n, k = np.nonzero(topk_g == e)
        pairs = (n * (used + 1) + k).tolist()
        for c in range(0, len(pairs), entry_cols):
            entries.append((e, len(cols) + c, min(entry_cols, len(pairs) - c)))
        cols += pairs
    own = [gathered_row(rank, rows, i) * (used + 1) + used for i in range(rows)]
    for c in range(0, rows, entry_cols):
        entries.append((-1, len(cols) + c, min(entry_cols, rows - c)))
    cols += own
    return entries, np.asarray(cols, dtype=np.int64)


def pair_destination(pair, rows, used):
    """(owner rank, row of the owner's `down` buffer) of a pair's output: the rank that owns the pair's ROW
    keeps (used + 1) output rows per local row, in slot order."""
    per_rank = rows * (used + 1)
    return int(pair // per_rank), int(pair % per_rank)


def connect(graph, rank, world, all_gather_bytes):
    """One process per GPU: exports this rank's exchange buffers, swaps the handles through
    `all_gather_bytes(bytes) -> [bytes] * world` (torch.distributed or any other transport), maps the peers
    and switches expert parallelism on."""
    mine = graph.ep_export(rank, world)
    handles = all_gather_bytes(mine)
    if len(handles) != world or handles[rank] != mine:
        raise RuntimeError("ep.connect: the gathered handles are not in rank order")
    graph.ep_attach(handles)
    graph.ep_enable(True)
