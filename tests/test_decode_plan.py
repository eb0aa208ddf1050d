"""The flash-decode work partition (csrc/flash_decode_plan.h) replayed on the CPU: every tile is visited
once, every (sequence, kv head) unit is finished exactly once, merge records never collide."""
import ctypes as C
import random
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
CSRC = REPO / "llama3-custom-inference_b200" / "csrc"


@pytest.fixture(scope="module")
def plan(tmp_path_factory):
    so = tmp_path_factory.mktemp("plan") / "plan_harness.so"
    subprocess.run(["g++", "-O1", "-std=c++17", "-shared", "-fPIC", "-I", str(CSRC),
                    str(REPO / "tests" / "plan_harness.cpp"), "-o", str(so)], check=True)
    lib = C.CDLL(str(so))
    lib.plan_simulate.argtypes = [C.c_int] * 4 + [C.POINTER(C.c_int)] + [C.c_int] * 2 + [C.POINTER(C.c_int), C.POINTER(C.c_longlong)]
    lib.plan_static.argtypes = [C.c_int] * 7 + [C.POINTER(C.c_int), C.POINTER(C.c_int)]
    return lib


def static_deal(plan, B, Hq, Hkv, D, n_seq, ragged=False, sms=148, max_clusters=(72, 34, 14)):
    """(goes to the static kernel, W warps per unit, C CTAs per unit, CTAs) on a device with `sms` SMs that holds
    `max_clusters` clusters of 2, 4, 8 CTAs at once."""
    out = (C.c_int * 3)()
    takes = plan.plan_static(B, Hq, Hkv, D, n_seq, int(ragged), sms, (C.c_int * 3)(*max_clusters), out)
    return bool(takes), out[0], out[1], out[2]


def simulate(plan, B, Hkv, D, n_seq, lens, G, stages=3):
    info = (C.c_int * 4)()
    stats = (C.c_longlong * 7)()
    arr = (C.c_int * B)(*lens) if lens is not None else None
    rc = plan.plan_simulate(B, Hkv, D, n_seq, arr, G, stages, info, stats)
    assert rc == 0, f"invariant {rc} broken: info={list(info)} B={B} Hkv={Hkv} D={D} n_seq={n_seq} lens={lens} G={G}"
    return list(stats)


def test_constants(plan):
    assert plan.plan_tile_tokens(128) == 16 and plan.plan_tile_tokens(64) == 32
    assert [plan.plan_head_group(h) for h in (1, 2, 3, 4, 6, 8, 12, 32)] == [1, 2, 1, 4, 2, 8, 4, 8]
    assert plan.plan_max_ctas(148, 8) == 148 and plan.plan_max_ctas(148, 1) == 1184


def test_ranges_are_balanced_and_invertible(plan):
    for total, G in [(1, 1), (3, 8), (300, 148), (148, 148), (149, 148), (65536, 148), (12288, 148), (7, 1184)]:
        sizes = [plan.plan_range_begin(c + 1, total, G) - plan.plan_range_begin(c, total, G) for c in range(G)]
        assert sum(sizes) == total and max(sizes) - min(sizes) <= 1
        for col in range(0, total, max(1, total // 97)):
            c = plan.plan_cta_of(col, total, G)
            assert plan.plan_range_begin(c, total, G) <= col < plan.plan_range_begin(c + 1, total, G)


@pytest.mark.parametrize("B,Hkv,D,n_seq,G", [
    (1, 8, 64, 256, 8),          # config 1
    (1, 8, 128, 131072, 148),    # config 3
    (64, 8, 64, 2176, 148),      # end-to-end decode batch
    (1, 8, 128, 1, 1), (1, 8, 128, 17, 2), (2, 1, 64, 100, 1184), (3, 2, 128, 777, 592),
    (5, 32, 128, 333, 148), (4, 6, 64, 65, 592), (2, 3, 128, 4096, 1184), (7, 4, 64, 31, 296),
])
def test_uniform_lengths(plan, B, Hkv, D, n_seq, G):
    stats = simulate(plan, B, Hkv, D, n_seq, None, G)
    assert stats[0] + stats[1] == B * Hkv
    if stats[6]:
        assert stats[1] == 0      # whole units per CTA: nothing to merge
    else:
        assert stats[3] - stats[4] <= 1


def test_config2_ragged_batch(plan):
    rng = random.Random(42)
    lens = [rng.randint(1024, 2048) for _ in range(16)]
    stats = simulate(plan, 16, 8, 128, 2048, lens, 148)
    assert stats[6] == 0 and stats[0] + stats[1] == 16 * 8 and stats[3] - stats[4] <= 1
    assert stats[5] == sum((l + 15) // 16 for l in lens)


def test_random_ragged_batches(plan):
    rng = random.Random(7)
    for _ in range(300):
        B = rng.randint(1, 40)
        Hkv = rng.choice([1, 2, 3, 4, 6, 8, 16])
        D = rng.choice([64, 128])
        n_seq = rng.choice([1, 15, 16, 17, 63, 64, 65, 200, 1000])
        lens = [rng.choice([0, 1, n_seq, rng.randint(0, n_seq), rng.randint(-3, n_seq + 5)]) for _ in range(B)]
        hg = plan.plan_head_group(Hkv)
        G = rng.choice([1, 2, 3, 7, 148, plan.plan_max_ctas(148, hg)])
        stats = simulate(plan, B, Hkv, D, n_seq, lens, G, stages=rng.choice([1, 2, 3, 4]))
        assert stats[0] + stats[1] == B * Hkv


def test_short_sequences_are_not_cut(plan):
    # the start of an end-to-end decode: 64 sequences of ~150 tokens in a cache padded to 2176
    rng = random.Random(11)
    lens = [rng.randint(129, 180) for _ in range(64)]
    stats = simulate(plan, 64, 8, 64, 2176, lens, 148)
    assert stats[6] == 1 and stats[1] == 0 and stats[0] == 64 * 8
    # late in the same decode the sequences are long and are cut again
    stats = simulate(plan, 64, 8, 64, 2176, [2100] * 64, 148)
    assert stats[6] == 0
    # one long sequence is always cut
    assert simulate(plan, 1, 8, 128, 131072, None, 148)[6] == 0


# ---- the static deal (flash_decode_small.cu): split and choice of kernel from host-side sizes ---------------------

def test_static_split_of_the_benchmark_shapes(plan):
    assert static_deal(plan, 1, 32, 8, 64, 256) == (True, 8, 1, 8)              # config 1: 8 tiles, no cluster
    assert static_deal(plan, 16, 32, 8, 128, 2048, ragged=True) == (True, 8, 1, 128)   # config 2
    assert static_deal(plan, 1, 32, 8, 128, 131072) == (True, 8, 8, 64)         # config 3: clusters of 8, 12-warp shape
    assert static_deal(plan, 1, 32, 8, 128, 262144)[0] is False                 # twice that: persistent kernel
    assert static_deal(plan, 64, 32, 8, 64, 2176) == (True, 2, 1, 128)          # decode batch: 4 units per CTA
    assert static_deal(plan, 64, 32, 8, 64, 2176, ragged=True)[0] is False      # ... unless the lengths may differ
    assert static_deal(plan, 1, 32, 8, 128, 16384) == (True, 8, 8, 64)          # few long units: clusters of 8
    assert static_deal(plan, 2, 32, 8, 128, 2048) == (True, 8, 4, 64)           # 16 clusters of 8 would not fit
    assert static_deal(plan, 2, 32, 2, 128, 512)[0] is False                    # 16 query heads per KV head
    assert static_deal(plan, 1, 32, 8, 64, 131072)[0] is True                   # long runs: the 12-warp shape keeps up
    assert static_deal(plan, 200, 8, 8, 64, 128)[0] is False                    # 1600 units: more than one wave
    assert static_deal(plan, 16, 32, 8, 128, 8192) == (True, 8, 1, 128)         # 4 MB per CTA: level with the persistent kernel
    assert static_deal(plan, 16, 32, 8, 128, 16384)[0] is False                 # 8 MB per CTA at the shared memory rate


def test_static_split_invariants(plan):
    rnd = random.Random(7)
    for _ in range(3000):
        B, Hkv = rnd.choice([1, 2, 3, 5, 8, 16, 40, 64, 150]), rnd.choice([1, 2, 3, 4, 8])
        D, n_seq = rnd.choice([64, 128]), rnd.choice([1, 31, 32, 100, 511, 512, 513, 2048, 5000, 40000, 131072])
        sms = rnd.choice([148, 132, 20])
        mc = (rnd.choice([0, sms // 2 - 2]), rnd.choice([0, sms // 4 - 3]), rnd.choice([0, 3, sms // 8 - 4]))
        takes, W, Cc, ctas = static_deal(plan, B, Hkv * rnd.choice([1, 4, 8]), Hkv, D, n_seq, rnd.random() < 0.5, sms, mc)
        units, tiles = B * Hkv, -(-n_seq // (16 if D == 128 else 32))
        assert W in (1, 2, 4, 8) and Cc in (1, 2, 4, 8) and (Cc == 1 or W == 8)
        if ctas == 0:
            assert not takes and units > 8 * sms
            continue
        assert ctas <= sms and ctas == -(-units // (8 // W)) * Cc          # one wave, every unit placed
        if Cc > 1:
            assert tiles >= 8 * Cc and tiles >= 32                           # every warp of the cluster has a tile
            assert units <= mc[{2: 0, 4: 1, 8: 2}[Cc]]                       # all clusters resident at once
        if W < 8:
            assert -(-units // (8 // W // 2)) > sms                          # half as many units per CTA would not fit
        if takes:
            share = n_seq * 4 * D * (8 // W) / Cc
            assert share <= 9e6
