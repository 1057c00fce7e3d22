"""Model check of the rule that lets packet generations (and staging halves) alternate without trailing barriers.

The device kernels write into their peers' inboxes right when they start, into the generation chosen by the parity
of the call number, and never reset anything. That is only safe if a rank cannot reach call m+2 while some peer still
reads generation m. The library's rule is: a rank leaves call m only when it knows that every rank has ENTERED call m.
All-to-all kernels give that for free; rooted kernels (broadcast: receivers hear only from the root; reduce: senders
hear from nobody) need the entry announcements that csrc/kernels/ll_collectives.cu sends.

This test explores every interleaving of a small abstract model (3 ranks, 3 calls) and checks that
  * with the announcements no call sequence over {all-reduce, broadcast, reduce} can overwrite an unread packet,
  * without them (and with acknowledgements to the root only) the sequence all-reduce, broadcast, all-reduce can.
No GPU is involved; the model is the protocol, not the kernels.
"""
import itertools

N = 3   # ranks


def plan(kind, root, rank):
    """(peers whose inbox I write when I start, peers whose packet I read)."""
    others = [p for p in range(N) if p != rank]
    if kind == "allreduce":
        return others, others
    if kind == "broadcast":
        return (others, []) if rank == root else ([], [root])
    if kind == "reduce":
        return ([], others) if rank == root else ([root], [])
    raise ValueError(kind)


def explore(calls, announce):
    """Depth-first search over all interleavings. A rank's steps within a call: write (all targets at once, plus the
    entry announcement), then one step per packet it reads (each possible once the source has written for this call),
    then leave (possible once all reads are done and, with `announce`, everybody has entered this call; without it the
    root of a broadcast waits until the receivers have read, the senders of a reduce until the root has read).
    Returns a violation description, "deadlock" when no interleaving finishes all calls, or None."""
    K = len(calls)
    # state: per rank (call index, wrote?, frozenset of sources read)
    start = tuple((0, False, frozenset()) for _ in range(N))
    # inbox[(owner, gen, src)] = call number of the packet lying there (or -1)
    seen = set()
    finished = False
    stack = [(start, tuple())]
    while stack:
        ranks, inbox_items = stack.pop()
        key = (ranks, inbox_items)
        if key in seen:
            continue
        seen.add(key)
        inbox = dict(inbox_items)
        if all(m >= K for m, _, _ in ranks):
            finished = True
        for r in range(N):
            m, wrote, read = ranks[r]
            if m >= K:
                continue
            kind, root = calls[m]
            targets, sources = plan(kind, root, r)
            if not wrote:
                # the write step: check that no target still has an unread packet of mine from call m-2 in this generation
                new_inbox = dict(inbox)
                for t in targets:
                    slot = (t, m % 2, r)
                    old = inbox.get(slot, -1)
                    if old >= 0:
                        tm, _, tread = ranks[t]
                        still_needed = tm == old and r in plan(*calls[old], t)[1] and r not in tread
                        if tm < old or still_needed:
                            return "rank %d in call %d overwrites the packet of call %d that rank %d (in call %d) has not read" % (r, m, old, t, tm)
                    new_inbox[slot] = m
                nxt = list(ranks)
                nxt[r] = (m, True, read)
                stack.append((tuple(nxt), tuple(sorted(new_inbox.items()))))
                continue
            progressed = False
            for s in sources:
                if s in read:
                    continue
                if inbox.get((r, m % 2, s), -1) == m:       # the packet of this call has arrived
                    nxt = list(ranks)
                    nxt[r] = (m, True, read | {s})
                    stack.append((tuple(nxt), inbox_items))
                    progressed = True
                elif inbox.get((r, m % 2, s), -1) > m:
                    return "rank %d in call %d finds a packet of call %d from rank %d where it expects its own call" % (r, m, inbox[(r, m % 2, s)], s)
            if progressed or set(sources) - read:
                continue
            # all packets read: may I leave?
            def entered(p):
                pm, pw, _ = ranks[p]
                return pm > m or (pm == m and pw)
            def has_read_from(p, src):
                pm, _, pread = ranks[p]
                return pm > m or (pm == m and src in pread)
            if announce:
                ok = all(entered(p) for p in range(N) if p != r)
            elif kind == "broadcast" and r == root:
                ok = all(has_read_from(p, r) for p in range(N) if p != r)          # acknowledgements
            elif kind == "reduce" and r != root:
                ok = has_read_from(root, r)                                          # acknowledgement
            else:
                ok = True
            if ok:
                nxt = list(ranks)
                nxt[r] = (m + 1, False, frozenset())
                stack.append((tuple(nxt), inbox_items))
    return None if finished else "deadlock"


def all_sequences(length):
    kinds = [("allreduce", 0)] + [(k, root) for k in ("broadcast", "reduce") for root in range(N)]
    return itertools.product(kinds, repeat=length)


def test_entry_announcements_make_every_sequence_safe():
    for calls in all_sequences(3):
        assert explore(list(calls), announce=True) is None, calls


def test_acknowledging_the_root_only_is_not_enough():
    bad = explore([("allreduce", 0), ("broadcast", 0), ("allreduce", 0)], announce=False)
    assert bad is not None and "overwrites" in bad, bad
    # and the all-to-all kernels alone never needed anything extra
    assert explore([("allreduce", 0)] * 3, announce=False) is None
