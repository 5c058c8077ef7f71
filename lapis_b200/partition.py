"""Row-block partitioning of a CSR matrix over several GPUs (host-side integer logic).

The reference has no multi-device path (its PartTensor dialect only plans
partitions and ships no communication code), so the rule is this package's own:
contiguous row blocks with equal numbers of stored entries,

    bounds[g] = first row whose start offset is >= pos[0] + g*nnz/G,   g = 0..G-1
    bounds[G] = nrows

Rank g owns rows [bounds[g], bounds[g+1]) with their slice of crd/val, offsets
rebased to start at 0.  For operators whose input vector is also distributed (the
PCG solve) each rank reads a contiguous *window* of the vector -- its own entries
plus the halo its columns reach -- and the pieces of that window owned by other
ranks are what the halo exchange moves.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ._lib import check, load


def partition_rows(pos: np.ndarray, G: int) -> np.ndarray:
    """nnz-balanced row bounds (int64[G+1]), computed by the C library."""
    pos = np.ascontiguousarray(pos)
    if pos.dtype not in (np.int32, np.int64):
        raise TypeError("pos must be int32 or int64")
    bounds = np.empty(G + 1, dtype=np.int64)
    check(load().lapis_b200_partition_rows(pos.itemsize, len(pos) - 1, pos.ctypes.data_as(ctypes.c_void_p), G,
                                           bounds.ctypes.data_as(ctypes.c_void_p)))
    return bounds


def row_block(pos, crd, val, r0: int, r1: int):
    """Rows [r0, r1) as a CSR of their own: offsets rebased to 0, global column indices."""
    lo, hi = int(pos[r0]), int(pos[r1])
    lpos = (pos[r0:r1 + 1] - pos[r0]).astype(pos.dtype)
    return lpos, crd[lo:hi], val[lo:hi]


def column_window(crd_local: np.ndarray, r0: int, r1: int):
    """Smallest contiguous column range [c0, c1) that holds the block's own rows [r0, r1)
    and every column its entries reference."""
    if crd_local.size == 0:
        return int(r0), int(r1)
    return min(int(r0), int(crd_local.min())), max(int(r1), int(crd_local.max()) + 1)


def exchange_plan(bounds: np.ndarray, windows):
    """Halo pieces per rank for windows[g] = (c0, c1).

    Returns ``recv[g]`` = list of (owner, start, stop) global index ranges rank g needs from
    other owners, and ``send[g]`` = list of (consumer, start, stop) it must provide; both
    sorted by peer then start, so that matching sends and receives pair up in order.
    """
    G = len(bounds) - 1
    recv = [[] for _ in range(G)]
    send = [[] for _ in range(G)]
    for g, (c0, c1) in enumerate(windows):
        for o in range(G):
            if o == g:
                continue
            s, e = max(c0, int(bounds[o])), min(c1, int(bounds[o + 1]))
            if s < e:
                recv[g].append((o, s, e))
                send[o].append((g, s, e))
    for lst in send:
        lst.sort()
    return recv, send


def push_pieces(send, windows, rank: int, peer_window_len, peer_p_index, work_addr, mbox_addr, halo_index: int):
    """Records for the peer-memory halo push of a row-partitioned PCG (consumed by
    ``lapis_b200_pcg_p2p_halo_push``): for every (consumer, start, stop) of ``send`` the four integers
    {destination address of the piece inside the consumer's p window, offset of the piece in this rank's
    window, length, address of this rank's halo flag in the consumer's mailbox}.

    ``windows[g] = (c0, c1)`` are the ranks' column windows, ``peer_window_len[g]`` / ``peer_p_index[g]`` the
    length of rank g's window and the index (in doubles) of its first element inside g's workspace,
    ``work_addr[g]`` / ``mbox_addr[g]`` the addresses at which this rank sees g's workspace and mailbox.
    Every piece is checked against both windows: no address is formed that was not bounded first.
    """
    c0_me, c1_me = windows[rank]
    out = []
    for (consumer, s, e) in send:
        c0_peer = windows[consumer][0]
        dst_off, src_off, length = s - c0_peer, s - c0_me, e - s
        if not (length > 0 and 0 <= dst_off and dst_off + length <= peer_window_len[consumer]
                and 0 <= src_off and src_off + length <= c1_me - c0_me):
            raise RuntimeError(f"halo piece [{s}, {e}) for rank {consumer} lies outside a window")
        out += [work_addr[consumer] + 8 * (peer_p_index[consumer] + dst_off), src_off, length,
                mbox_addr[consumer] + 8 * (halo_index + rank)]
    return out
