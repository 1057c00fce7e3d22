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


# ---------------------------------------------------------------------------------------------------------------------
# grouped send / recv: FIFO credits and the batching of long groups
# ---------------------------------------------------------------------------------------------------------------------

def run_group(ops_per_rank, batch, depth, partition):
    """Fixpoint simulation of one grouped call (csrc/kernels/p2p.cu, GpuCommImpl::p2p_launch).

    ops_per_rank[r] is the recorded list of ("send" | "recv", peer, chunks). Chunk numbers per ordered pair are given
    out in recording order. The list is cut into launches of `batch` operations; a rank starts its next launch when
    all operations of the current one are done; inside a launch all operations progress concurrently. A sender may
    write chunk G when G < depth or the receiver has consumed chunk G - depth; a receiver may read chunk G once it is
    written. `partition`: "batch" moves the receives of every launch to its front (what the library does), "global"
    moves all receives of the whole group to the front before cutting (the mistake this test guards against),
    "none" keeps the recording order. Returns True when every operation completes, False on deadlock."""
    n = len(ops_per_rank)
    next_chunk = {}
    plans = []
    for r, ops in enumerate(ops_per_rank):
        tagged = []
        for kind, peer, chunks in ops:
            key = (r, peer) if kind == "send" else (peer, r)
            first = next_chunk.get((kind, key), 0)
            next_chunk[(kind, key)] = first + chunks
            tagged.append([kind, key, first, chunks, 0])            # ..., chunks done
        if partition == "global":
            tagged.sort(key=lambda o: o[0] != "recv")
        launches = [tagged[i:i + batch] for i in range(0, len(tagged), batch)]
        if partition == "batch":
            for launch in launches:
                launch.sort(key=lambda o: o[0] != "recv")
        plans.append(launches)
    written, consumed = {}, {}                                       # per ordered pair: chunks written / consumed
    current = [0] * n
    while True:
        progress = False
        for r in range(n):
            if current[r] >= len(plans[r]):
                continue
            launch = plans[r][current[r]]
            for op in launch:
                kind, key, first, chunks, done = op
                while done < chunks:
                    g = first + done
                    if kind == "send":
                        if g >= depth and consumed.get(key, 0) < g - depth + 1:
                            break
                        if written.get(key, 0) != g:                 # chunks of one pair are written in order
                            break
                        written[key] = g + 1
                    else:
                        if written.get(key, 0) < g + 1 or consumed.get(key, 0) != g:
                            break
                        consumed[key] = g + 1
                    done += 1
                    progress = True
                op[4] = done
            if all(op[4] == op[3] for op in launch):
                current[r] += 1
                progress = True
        if all(current[r] >= len(plans[r]) for r in range(n)):
            return True
        if not progress:
            return False


def ring(n, window, chunks):
    return [[op for _ in range(window) for op in (("send", (r + 1) % n, chunks), ("recv", (r - 1) % n, chunks))] for r in range(n)]


def all_to_all(n, chunks):
    return [[("recv", (r - k) % n, chunks) for k in range(1, n)] + [("send", (r + k) % n, chunks) for k in range(1, n)] for r in range(n)]


def test_grouped_send_recv_never_deadlocks_with_receivers_first_per_launch():
    for n in (2, 3, 8):
        for chunks in (1, 3, 9):                                     # 9 > FIFO depth: senders need credit
            assert run_group(all_to_all(n, chunks), batch=16, depth=4, partition="batch")
            for window in (1, 4, 10):
                assert run_group(ring(n, window, chunks), batch=16, depth=4, partition="batch"), (n, window, chunks)
                assert run_group(ring(n, window, chunks), batch=16, depth=4, partition="none"), (n, window, chunks)
    # gather / scatter: the root groups n-1 operations, everybody else issues a single one
    n = 8
    gather = [[("recv", p, 5) for p in range(1, n)]] + [[("send", 0, 5)] for _ in range(1, n)]
    assert run_group(gather, batch=16, depth=4, partition="batch")


def test_moving_all_receives_of_a_long_group_to_the_front_would_deadlock():
    # 10 sends and 10 receives per rank = 20 operations = two launches: with all receives first, the receives of the
    # first launch wait for sends that sit in the peers' second launch
    assert not run_group(ring(4, 10, 1), batch=16, depth=4, partition="global")
    assert run_group(ring(4, 10, 1), batch=16, depth=4, partition="batch")


# ---------------------------------------------------------------------------------------------------------------------
# pipelined switch broadcast / reduce: chunk and CTA ranges (csrc/kernels/nvls_rooted.cu, csrc/device/geometry.cuh)
# ---------------------------------------------------------------------------------------------------------------------

def rooted_ranges(count, es, nchunks, G):
    """[(chunk, cta, first element, one past the last)] as the kernel computes them: the message is cut into nchunks
    pieces of whole 16-byte vectors, every piece into G CTA ranges of whole vectors."""
    VE = 16 // es
    roundup = lambda x, m: (x + m - 1) // m * m
    chunk = roundup((count + nchunks - 1) // nchunks, VE)
    out = []
    for k in range(nchunks):
        base = k * chunk
        cnt = 0 if base >= count else min(count - base, chunk)
        for g in range(G):
            per = cnt                                            # GEO_WHOLE: one shard holding the chunk
            epb = roundup((per + G - 1) // G, VE)
            blo = min(epb * g, per)
            bhi = min(blo + epb, per)
            lo, hi = min(blo, cnt), min(bhi, cnt)
            out.append((k, g, base + lo, base + hi))
    return out


def rooted_chunks(nbytes):
    return max(2, min(24, (nbytes + (8 << 20) - 1) // (8 << 20)))


def test_pipelined_switch_broadcast_ranges_cover_the_message_once():
    for es in (1, 2, 4, 8):
        for count in [1, 15, 16, 17, 4099, (1 << 20) + 3, (24 << 20) // es + 5, (200 << 20) // es + 1]:
            nchunks = rooted_chunks(count * es)
            for G in (1, 7, 16, 72):
                ranges = [(lo, hi) for _, _, lo, hi in rooted_ranges(count, es, nchunks, G) if hi > lo]
                ranges.sort()
                assert ranges[0][0] == 0 and ranges[-1][1] == count, (es, count, G)
                for (a, b), (c, d) in zip(ranges, ranges[1:]):
                    assert b == c, ("gap or overlap", es, count, G, (a, b), (c, d))
                # every range starts on a 16-byte boundary of the message (what multimem.st needs when the buffer is aligned)
                assert all((lo * es) % 16 == 0 for lo, _ in ranges), (es, count, G)
