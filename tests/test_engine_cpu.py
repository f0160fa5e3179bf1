"""Promotion engine against host memory (device = -1): ordering of bytes -> row -> sequence number, the host cache
(hits, eviction), cancellation, failing and slow drives, the RAM tier and the two-drive split.  The failures are made
on the host side (a record index past the end of the file, the engine's own fault switches), as the reference's
streaming/smoke_fault.py does; no GPU is involved."""
import ctypes as C
import os
import time

import numpy as np
import pytest

REC = 8192          # record size (a multiple of 4096)
NREC = 24


@pytest.fixture(scope="module")
def record_file(tmp_path_factory):
    from nestquant_b200 import build
    build.build()
    d = tmp_path_factory.mktemp("rec")
    rng = np.random.default_rng(7)
    data = rng.integers(0, 256, size=(NREC, REC), dtype=np.uint8)
    for name in ("rank0.bin", "rank0_copy.bin"):
        data.tofile(os.path.join(d, name))
    return str(d), data


class Target:
    """host-memory stand-ins for the device side: slots, the staged table and the sequence numbers"""

    def __init__(s, nslot, E=16):
        s.slots = np.zeros((nslot, REC), dtype=np.uint8)
        s.stage = np.zeros((E, 20), dtype=np.int64)
        s.seq = np.zeros(E, dtype=np.int32)

    def slot_ptr(s, i):
        return s.slots[i].ctypes.data

    def stage_ptr(s, e):
        return s.stage[e].ctypes.data

    def seq_ptr(s, e):
        return s.seq[e:e + 1].ctypes.data


def drain(eng, n, timeout=10.0):
    out, t0 = [], time.time()
    while len(out) < n and time.time() - t0 < timeout:
        out += eng.poll()
        time.sleep(0.002)
    assert len(out) == n, (len(out), n, eng.stats())
    return out


def test_upgrade_writes_bytes_row_and_sequence_number(record_file):
    from nestquant_b200.engine import Engine
    d, data = record_file
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 4, 2, -1), Target(4)
    for i, rec in enumerate((5, 0, 23)):
        eng.upgrade(100 + i, rec, T.slot_ptr(i), T.stage_ptr(i), [rec * 10 + k for k in range(20)], T.seq_ptr(i), i + 1)
    res = drain(eng, 3)
    assert sorted(t for t, *_ in res) == [100, 101, 102]
    for i, rec in enumerate((5, 0, 23)):
        assert np.array_equal(T.slots[i], data[rec])
        assert T.stage[i].tolist() == [rec * 10 + k for k in range(20)] and T.seq[i] == i + 1
    assert all(not hit and 0 <= tr <= te for _, hit, tr, te in res)
    st = eng.stats()
    assert st["upgrades"] == 3 and st["bytes_read"] == 3 * REC and st["host_hits"] == 0 and st["drive_reads"] == [3]
    eng.post(200, T.stage_ptr(0), [7] * 20, T.seq_ptr(0), 9)              # demotion: row and sequence number only
    (tag, hit, tr, te), = drain(eng, 1)
    assert tag == 200 and T.stage[0].tolist() == [7] * 20 and T.seq[0] == 9 and np.array_equal(T.slots[0], data[5])
    assert eng.stats()["posts"] == 1
    eng.close()


def test_host_cache_hits_and_evicts_least_recently_used(record_file):
    from nestquant_b200.engine import Engine
    d, data = record_file
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 3, 1, -1), Target(2)
    seq = 0

    def up(rec):
        nonlocal seq
        seq += 1
        eng.upgrade(seq, rec, T.slot_ptr(0), T.stage_ptr(0), [0] * 20, T.seq_ptr(0), seq)
        (_, hit, _, _), = drain(eng, 1)
        assert np.array_equal(T.slots[0], data[rec])
        return hit

    assert [up(r) for r in (1, 2, 3)] == [False, False, False]
    assert up(1) is True                       # still cached; now the most recently used
    assert up(4) is False                      # evicts record 2 (least recently used)
    assert up(1) is True and up(3) is True and up(2) is False
    st = eng.stats()
    assert st["host_hits"] == 3 and st["bytes_read"] == 5 * REC
    eng.close()


def test_failed_read_never_posts_the_row(record_file):
    from nestquant_b200.engine import Engine
    d, data = record_file
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 2, 1, -1), Target(1)
    eng.upgrade(1, NREC + 3, T.slot_ptr(0), T.stage_ptr(0), [5] * 20, T.seq_ptr(0), 1)     # past the end of the file
    (tag, hit, tr, te), = drain(eng, 1)
    assert tag == 1 and not hit and tr < 0 and te == -1.0
    assert T.seq[0] == 0 and not T.stage[0].any()
    eng.upgrade(2, 3, T.slot_ptr(0), T.stage_ptr(0), [6] * 20, T.seq_ptr(0), 2)            # the engine keeps working
    (tag, hit, tr, te), = drain(eng, 1)
    assert tag == 2 and tr >= 0 and T.seq[0] == 2 and np.array_equal(T.slots[0], data[3])
    eng.close()


def test_failing_drive_switch(record_file, monkeypatch):
    from nestquant_b200.engine import Engine
    d, _ = record_file
    monkeypatch.setenv("NQ_FAULT_FAIL_PPM", "1000000")
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 2, 2, -1), Target(2)
    for i in range(4):
        eng.upgrade(i, i, T.slot_ptr(i % 2), T.stage_ptr(i), [1] * 20, T.seq_ptr(i), 1)
    res = drain(eng, 4)
    assert all(not hit and tr < 0 and te == -1.0 for _, hit, tr, te in res)
    assert not T.seq.any() and eng.stats()["fault_injected"] == 4
    eng.close()


def test_cancel_drops_only_operations_that_have_not_started(record_file, monkeypatch):
    from nestquant_b200.engine import Engine
    d, data = record_file
    monkeypatch.setenv("NQ_FAULT_READ_MS", "150")                       # a slow drive: one read every 150 ms
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 2, 1, -1), Target(4)
    for i in range(4):
        eng.upgrade(i, i, T.slot_ptr(i), T.stage_ptr(i), [i] * 20, T.seq_ptr(i), 1)
    time.sleep(0.03)
    eng.cancel(3); eng.cancel(0)                                         # 0 has already started, 3 is still waiting
    res = {t: (hit, tr, te) for t, hit, tr, te in drain(eng, 4)}
    assert res[3] == (False, -1e9, -1e9) and T.seq[3] == 0
    assert res[0][1] >= 0 and T.seq[0] == 1 and np.array_equal(T.slots[0], data[0])
    assert T.seq[1] == 1 and T.seq[2] == 1
    assert eng.stats()["cancelled"] == 1
    eng.close()


def test_ram_tier_serves_its_records_and_can_be_dropped(record_file):
    from nestquant_b200.engine import Engine
    d, data = record_file
    eng, T = Engine(os.path.join(d, "rank0.bin"), REC, 2, 1, -1), Target(1)
    assert eng.tier_load([7, 9, 11]) == 3
    with pytest.raises(RuntimeError):
        eng.tier_load([1])
    eng.upgrade(1, 9, T.slot_ptr(0), T.stage_ptr(0), [0] * 20, T.seq_ptr(0), 1)
    (_, hit, _, _), = drain(eng, 1)
    assert hit and np.array_equal(T.slots[0], data[9])
    st = eng.stats()
    assert st["tier_hits"] == 1 and st["tier_bytes"] == REC and st["bytes_read"] == 0 and st["tier_state"] == 1 and st["tier_recs"] == 3
    eng.tier_drop()
    t0 = time.time()
    while eng.stats()["tier_state"] != 3 and time.time() - t0 < 5:
        time.sleep(0.005)
    assert eng.stats()["tier_state"] == 3
    eng.upgrade(2, 9, T.slot_ptr(0), T.stage_ptr(0), [0] * 20, T.seq_ptr(0), 2)           # now from the drive
    (_, hit, _, _), = drain(eng, 1)
    assert not hit and eng.stats()["bytes_read"] == REC
    eng.close()


def test_two_drives_share_the_reads(record_file):
    from nestquant_b200.engine import Engine
    d, data = record_file
    eng = Engine(os.path.join(d, "rank0.bin"), REC, 8, 2, -1, alt_path=os.path.join(d, "rank0_copy.bin"), qd_alt=2)
    T = Target(8)
    for i in range(16):
        eng.upgrade(i, i, T.slot_ptr(i % 8), T.stage_ptr(i % 16), [i] * 20, T.seq_ptr(i % 16), 1)
        if i % 8 == 7:
            drain(eng, 8)
    st = eng.stats()
    assert st["drives"] == 2 and sum(st["drive_reads"]) == 16 and sum(st["drive_bytes"]) == 16 * REC and st["drive_qd"] == [2, 2]
    assert np.array_equal(T.slots[7], data[15])
    eng.close()


def test_open_rejects_bad_arguments(record_file):
    from nestquant_b200.capi import NestQuantError
    from nestquant_b200.engine import Engine
    d, _ = record_file
    with pytest.raises(NestQuantError):
        Engine(os.path.join(d, "missing.bin"), REC, 2, 1, -1)
    with pytest.raises(NestQuantError):
        Engine(os.path.join(d, "rank0.bin"), REC + 1, 2, 1, -1)
    with pytest.raises(NestQuantError):
        Engine(os.path.join(d, "rank0.bin"), REC, 1, 2, -1)
