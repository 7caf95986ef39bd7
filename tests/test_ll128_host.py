"""CPU unit tests of the wire format, ring arithmetic, workspace layout and the protocol model.

The functions under test are the ones the device code calls (csrc/ll128.cuh, csrc/fifo.cuh),
compiled for the host.
"""
import ctypes
import random

import numpy as np
import pytest

RING_WORDS = 2048 * 16


def _ring():
    return np.full(RING_WORDS, 0xFFFFFFFFFFFFFFFF, dtype=np.uint64)


def _p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint64))


@pytest.fixture(scope="module")
def lib(host_lib):
    L = host_lib
    L.helix_flag_of.restype = ctypes.c_uint64
    L.helix_flag_of.argtypes = [ctypes.c_uint64]
    L.helix_ring_slot.restype = ctypes.c_uint32
    L.helix_ring_slot.argtypes = [ctypes.c_uint64]
    L.helix_chunk_ring_offset.restype = ctypes.c_uint32
    L.helix_chunk_ring_offset.argtypes = [ctypes.c_uint64, ctypes.c_int]
    for f in (L.helix_pack_message, L.helix_unpack_message):
        f.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64)]
    L.helix_pack_line.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.c_uint64, ctypes.c_int,
                                  ctypes.POINTER(ctypes.c_uint64)]
    L.helix_valid_prefix.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.c_uint64]
    L.helix_message_ready.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.c_uint64]
    L.helix_chunk_words.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.c_uint64, ctypes.c_int,
                                    ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
    L.helix_layout.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]
    for f in (L.helix_ring_offset, L.helix_sinfo_slot, L.helix_rinfo_slot):
        f.restype = ctypes.c_int64
        f.argtypes = [ctypes.c_int] * 4
    L.helix_ring_has_room.argtypes = [ctypes.c_uint64, ctypes.c_uint64]
    L.helix_model_run.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_int, ctypes.c_uint32, ctypes.POINTER(ctypes.c_int64)]
    return L


def test_line_counts(lib):
    # payload words -> lines: 15 data words per line
    assert lib.helix_lines_for_words(1) == 1
    assert lib.helix_lines_for_words(15) == 1
    assert lib.helix_lines_for_words(16) == 2
    assert lib.helix_lines_for_words(129) == 9      # MLA: 1024 B + 8 B
    assert lib.helix_lines_for_words(33) == 3       # GQA: 256 B + 8 B
    assert lib.helix_wire_bytes_for_words(129) == 1152
    # the reference's framing needs 1280 B / 512 B for the same messages
    assert lib.helix_wire_bytes_for_words(129) < 1280 and lib.helix_wire_bytes_for_words(33) < 512


def test_flags_never_collide_with_init_or_previous_lap(lib):
    assert lib.helix_flag_of(0) == 1
    for q in (0, 1, 2047, 2048, 10**12):
        f = lib.helix_flag_of(q)
        assert f != 0xFFFFFFFFFFFFFFFF and f != 0
        assert lib.helix_flag_of(q + 2048) != f
        assert lib.helix_ring_slot(q + 2048) == lib.helix_ring_slot(q)


@pytest.mark.parametrize("words", [1, 2, 15, 16, 33, 129, 257, 700])
@pytest.mark.parametrize("q0", [0, 5, 2040, 2047, 2048 * 7 + 2046])
def test_pack_unpack_roundtrip_with_wrap(lib, words, q0):
    rng = np.random.default_rng(words * 7919 + q0)
    payload = rng.integers(0, 2**63, size=words, dtype=np.uint64)
    ring = _ring()
    assert lib.helix_message_ready(_p(ring), words, q0) == 0
    lib.helix_pack_message(_p(payload), words, q0, _p(ring))
    assert lib.helix_message_ready(_p(ring), words, q0) == 1
    out = np.zeros(words, dtype=np.uint64)
    lib.helix_unpack_message(_p(ring), words, q0, _p(out))
    assert (out == payload).all()
    # a message at the same slots one lap later must not look ready
    assert lib.helix_message_ready(_p(ring), words, q0 + 2048) == 0


def test_partial_arrival_in_arbitrary_line_order(lib):
    words, q0 = 129, 2041           # wraps around the end of the ring
    nlines = lib.helix_lines_for_words(words)
    payload = np.arange(1, words + 1, dtype=np.uint64) * np.uint64(0x0101010101)
    ring = _ring()
    order = list(range(nlines))
    random.Random(3).shuffle(order)
    arrived = set()
    for j in order:
        lib.helix_pack_line(_p(payload), words, q0, j, _p(ring))
        arrived.add(j)
        prefix = lib.helix_valid_prefix(_p(ring), words, q0)
        expect = 0
        while expect in arrived:
            expect += 1
        assert prefix == expect
        assert lib.helix_message_ready(_p(ring), words, q0) == (1 if len(arrived) == nlines else 0)
    out = np.zeros(words, dtype=np.uint64)
    lib.helix_unpack_message(_p(ring), words, q0, _p(out))
    assert (out == payload).all()


def test_chunk_view_equals_line_view(lib):
    """What 8 lanes store (16 B each) is exactly the line the host packer writes."""
    words, q0 = 33, 2046
    payload = np.random.default_rng(0).integers(0, 2**63, size=words, dtype=np.uint64)
    ring = _ring()
    lib.helix_pack_message(_p(payload), words, q0, _p(ring))
    ring2 = _ring()
    lo, hi = ctypes.c_uint64(), ctypes.c_uint64()
    for ch in range(lib.helix_lines_for_words(words) * 8):
        lib.helix_chunk_words(_p(payload), words, q0, ch, ctypes.byref(lo), ctypes.byref(hi))
        off = lib.helix_chunk_ring_offset(q0, ch)
        assert off % 16 == 0
        ring2[off // 8] = lo.value
        ring2[off // 8 + 1] = hi.value
    assert (ring == ring2).all()


def test_chunk_map(lib):
    line, first, flag = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    seen = []
    for ch in range(24):
        lib.helix_chunk_map(ch, ctypes.byref(line), ctypes.byref(first), ctypes.byref(flag))
        assert line.value == ch // 8
        assert flag.value == (1 if ch % 8 == 7 else 0)
        seen.append(first.value)
        if not flag.value:
            seen.append(first.value + 1)
    assert seen == list(range(45))      # 3 lines x 15 payload words, each exactly once, in order


@pytest.mark.parametrize("cp", [1, 2, 4, 8, 16])
def test_layout(lib, cp):
    out = (ctypes.c_int64 * 6)()
    lib.helix_layout(cp, 148, out)
    max_c, ring_region, sinfo, rinfo, status, row = list(out)
    ref_ch = max(148 // (((cp + 7) // 8) * 2), 1)
    assert max_c == 2 * ref_ch
    assert row == 512 * 1024 * cp * ref_ch + 2 * 256 * cp * ref_ch
    assert ring_region == 256 * 1024 * cp * max_c
    assert sinfo == ring_region and rinfo > sinfo and status > rinfo and status + 256 <= row
    # slots do not overlap and stay inside their regions
    offs = set()
    for peer in range(cp):
        for c in (0, 1, max_c - 1):
            r = lib.helix_ring_offset(cp, 148, peer, c)
            assert r % (256 * 1024) == 0 and r + 256 * 1024 <= ring_region
            s = lib.helix_sinfo_slot(cp, 148, peer, c)
            t = lib.helix_rinfo_slot(cp, 148, peer, c)
            assert sinfo <= s < rinfo <= t < status
            offs.update([r, s, t])
    assert len(offs) == 3 * cp * 3 or max_c < 3


def test_entries_of_channel(lib):
    for entries in (0, 1, 5, 16, 149, 4096):
        for ch in (1, 3, 16, 148):
            tot = sum(lib.helix_entries_of_channel(entries, ch, c) for c in range(ch))
            assert tot == entries


def test_flow_control_rule(lib):
    assert lib.helix_ring_has_room(2047, 0) == 1
    assert lib.helix_ring_has_room(2048, 0) == 0
    assert lib.helix_ring_has_room(2048, 1) == 1
    assert lib.helix_ring_has_room(10**9 + 2047, 10**9) == 1


def _run_model(lib, cp, entries, words, channels, publish_every=0, drop=-1, seed=1):
    arr = (ctypes.c_int * len(entries))(*entries)
    moved = ctypes.c_int64()
    rc = lib.helix_model_run(cp, len(entries), arr, words, channels, publish_every, drop, seed, ctypes.byref(moved))
    return rc, moved.value


@pytest.mark.parametrize("cp", [2, 4, 8])
def test_model_many_small_calls_without_reinit(lib, cp):
    # many back-to-back calls of varying size; rings wrap several times, never re-initialised
    entries = [1, 3, 16, 2, 40, 7] * 40
    rc, moved = _run_model(lib, cp, entries, 129, 4, seed=cp)
    assert rc == 0
    assert moved == sum(entries) * 9 * cp * (cp - 1)


def test_model_single_call_larger_than_ring(lib):
    # 1200 messages x 9 lines on one channel = 5.3 ring laps in ONE call: needs in-call publishes
    rc, _ = _run_model(lib, 2, [1200], 129, 1, publish_every=32)
    assert rc == 0


def test_model_detects_deadlock_without_in_call_publish(lib):
    # same traffic, receiver publishes only at the end: the sender must stall (model reports 3)
    rc, _ = _run_model(lib, 2, [1200], 129, 1, publish_every=0)
    assert rc == 3


def test_model_dead_sender_is_detected(lib):
    rc, _ = _run_model(lib, 4, [8], 33, 2, drop=1)
    assert rc == 3


def _violations(host_lib, cp, outer, inner, mode, o_bytes, st_words, lse_scalar, strides, extents, has_st=1):
    import ctypes
    f = host_lib.helix_bounds_violations
    f.restype = ctypes.c_int
    ll = ctypes.c_longlong
    return f(cp, outer, inner, mode, o_bytes, st_words, lse_scalar, *[ll(x) for x in strides], *[ll(x) for x in extents],
             has_st)


def test_debug_bounds_checks_accept_the_bindings_strides_and_catch_wrong_ones(host_lib):
    """The per-message span checks of the exchange's debug mode, walked on the host over whole launches."""
    # combine mode, native layout: attn_out [B, H, D] bf16, lse [B, H] -> out [B, H/cp, D], global lse [B, H/cp]
    B, H, cp, D = 5, 16, 4, 128
    Hl = H // cp
    strides = [H * D * 2, Hl * D * 2, D * 2, H * 4, Hl * 4, 4, D * 2, 0, 0, 0]
    extents = [B * H * D * 2, B * H * 4, B * Hl * D * 2, B * Hl * 4]
    assert _violations(host_lib, cp, B, Hl, 1, D * 2, 1, 1, strides, extents) == 0
    bad = list(strides)
    bad[1] = Hl * D * 2 + 16                      # peer stride too long: the last peers' rows leave the tensor
    assert _violations(host_lib, cp, B, Hl, 1, D * 2, 1, 1, bad, extents) > 0
    bad = list(strides)
    bad[6] = D * 2 * 2                            # destination rows twice as far apart as the output is large
    assert _violations(host_lib, cp, B, Hl, 1, D * 2, 1, 1, bad, extents) > 0
    short = list(extents)
    short[1] -= 4                                 # LSE tensor one float short
    assert _violations(host_lib, cp, B, Hl, 1, D * 2, 1, 1, strides, short) == 1
    # exchange mode, the reference's layout: partial_o [E, cp, D], stats [E, cp, S]
    E, S = 7, 6
    strides = [cp * D * 2, D * 2, 0, cp * S * 4, S * 4, 0, cp * D * 2, D * 2, cp * S * 4, S * 4]
    extents = [E * cp * D * 2, E * cp * S * 4, E * cp * D * 2, E * cp * S * 4]
    assert _violations(host_lib, cp, E, 1, 0, D * 2, S // 2, 0, strides, extents) == 0
    extents[2] -= D * 2                           # output one row short: exactly the last (entry, peer) row is out
    assert _violations(host_lib, cp, E, 1, 0, D * 2, S // 2, 0, strides, extents) == 1
    # extents that were not recorded switch the check off
    assert _violations(host_lib, cp, E, 1, 0, D * 2, S // 2, 0, strides, [0, 0, 0, 0]) == 0
