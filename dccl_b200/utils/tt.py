"""Reader for the per-rank timestamp files (``.tt``) that ``Timestamp::flush`` writes:

    # number of entries:<N>
    # tag rank extra tsns
    <tag> <rank> <extra> <ts_ns>

(format of reference src/core/dccl.cpp:959-977).
"""

TAGS = {
    1000001: "WARMUP_START", 1000002: "WARMUP_END", 1000003: "TEST_START", 1000004: "TEST_END",
    1001001: "ALLREDUCE_ENTER", 1001020: "ALLREDUCE_MEMCPY", 1001021: "ALLREDUCE_RDH_PREPROCESS",
    1001030: "ALLREDUCE_REDUCESCATTER", 1001040: "ALLREDUCE_ALLGATHER", 1001041: "ALLREDUCE_RDH_POSTPROCESS",
    1001100: "ALLREDUCE_DONE", 1002001: "REDUCESCATTER_ENTER", 1002100: "REDUCESCATTER_DONE",
    1003001: "ALLGATHER_ENTER", 1003100: "ALLGATHER_DONE", 1004001: "BROADCAST_ENTER", 1004100: "BROADCAST_DONE",
    1005001: "REDUCE_ENTER", 1005100: "REDUCE_DONE", 1006001: "SEND_ENTER", 1006100: "SEND_DONE",
    1007001: "RECV_ENTER", 1007100: "RECV_DONE",
}


def read_tt(path):
    """Returns (declared_count, [(tag, rank, extra, ts_ns), ...])."""
    declared = None
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if line.startswith("#"):
                if "number of entries:" in line:
                    declared = int(line.split(":")[1])
                continue
            tag, rank, extra, ts = line.split()
            rows.append((int(tag), int(rank), int(extra), int(ts)))
    return declared, rows


def durations(rows, start_tag, end_tag):
    """Nanoseconds between each start_tag entry and the next end_tag entry."""
    out, t0 = [], None
    for tag, _rank, _extra, ts in rows:
        if tag == start_tag:
            t0 = ts
        elif tag == end_tag and t0 is not None:
            out.append(ts - t0)
            t0 = None
    return out
