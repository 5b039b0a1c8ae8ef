"""TEST INFRASTRUCTURE — NOT PRODUCT CODE.

Restatement, statement by statement in Python integers, of the residency plan of the reference's
Graph::plan_streaming (src/graph/memory.rs:64-125, 172-186): which parameters stay on the device
under a VRAM budget and which are streamed from host memory.  Parity is pinned by restatement
only: the reference has no test or vector for this function.
"""


def plan_streaming_layout(sizes, budget, reserve, pinned):
    """sizes: element count of every parameter tensor, indexed by tensor id (0 .. num_params-1).
    Returns the fields of StreamingReport (src/graph/memory.rs:7-14) as a dict."""
    sat_sub = lambda a, b: a - b if a > b else 0  # usize::saturating_sub
    pinned_set = set(pinned)
    pinned_vram = sum(sizes[p] * 4 * 4 for p in pinned)                      # :78-81
    budget_after_fixed = sat_sub(sat_sub(budget, reserve), pinned_vram)      # :83-85
    candidates = [i for i in range(len(sizes)) if i not in pinned_set]       # :87-88
    resident, streamed, used = [], [], 0
    for pid in candidates:                                                   # :95-103
        cost = sizes[pid] * 4 * 4
        if used + cost <= budget_after_fixed:
            used += cost
            resident.append(pid)
        else:
            streamed.append(pid)
    max_stream_bytes = max([sizes[p] * 4 for p in streamed], default=0)      # :105-109
    while max_stream_bytes > sat_sub(budget_after_fixed, used) and resident:  # :111-122
        # Iterator::max_by_key returns the last of several equally large elements
        best = 0
        for i in range(1, len(resident)):
            if sizes[resident[i]] >= sizes[resident[best]]:
                best = i
        pid = resident.pop(best)
        used -= sizes[pid] * 4 * 4
        streamed.append(pid)
    streamed_bytes = sum(sizes[p] * 4 for p in streamed)                     # :129-132
    resident_ids = list(pinned) + resident                                   # :180
    return {
        "resident_param_ids": resident_ids,
        "streamed_param_ids": streamed,
        "resident_bytes": sum(sizes[p] * 4 * 4 for p in resident_ids),       # :172-176
        "resident_headroom_bytes": 0,   # `let headroom = used;` is taken while used is still 0 (:92-93)
        "streamed_bytes": streamed_bytes,
        "streaming_headroom_bytes": max_stream_bytes,
    }
