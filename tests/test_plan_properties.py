"""Property-based tests of the plan compiler (no GPU): random algorithm / rank count / radix / batch / layout
against the direct-copy oracle, and an independent re-derivation of the radix bookkeeping of the Bruck family
(src/tuna2.cpp:24-44, src/twophase_tunable_rbruckv.cpp:22-60): a block that has to travel distance d is forwarded
once per non-zero base-r digit of d, by digit * r^x ranks each time."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from rbruck_alltoallv_b200 import Plan, host_alltoallv
from rbruck_alltoallv_b200.parallel.plan import ALGOS, HIERARCHICAL, LEADER_ROUTED
from rbruck_alltoallv_b200.utils import oracle

COMMON = dict(deadline=None, suppress_health_check=[HealthCheck.too_slow], max_examples=120)
BRUCK = ["rbruck", "rbruck_om", "tuna", "tuna2"]


@st.composite
def plan_args(draw):
    algo = draw(st.sampled_from(sorted(ALGOS)))
    P = draw(st.integers(1, 12))
    divisors = [d for d in range(1, P + 1) if P % d == 0]
    grouped = algo in HIERARCHICAL or algo in LEADER_ROUTED or algo.startswith("twolayer")
    n = draw(st.sampled_from(divisors)) if grouped else 0
    r = draw(st.integers(2, P + 1))
    return dict(algo=algo, P=P, n=n, r=r, r2=draw(st.integers(2, max(2, n + 1))), b=draw(st.integers(0, 4)),
                b2=draw(st.integers(0, 4)))


@settings(**COMMON)
@given(args=plan_args(), ts=st.sampled_from([1, 2, 4, 8, 16]), packed=st.booleans(), seed=st.integers(0, 2 ** 16),
       hi=st.integers(1, 40), zero_frac=st.floats(0.0, 0.6))
def test_any_valid_plan_moves_every_byte_to_its_place(args, ts, packed, seed, hi, zero_frac):
    plan = Plan(**args)
    if plan.err:
        # argument errors are the reference's codes: -1 bad radix / group size / non-power-of-two XOR, -2 group too large
        assert plan.err in (-1, -2), (args, plan.err)
        return
    P = args["P"]
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, hi + 1, size=(P, P))
    counts[rng.random((P, P)) < zero_frac] = 0
    if plan.uniform:
        counts[:] = hi
    prob = oracle.make_problem(counts, ts, seed, packed=packed)      # unpacked: shuffled blocks with holes between
    send = oracle.fill_send(prob, seed)
    recv = oracle.empty_recv(prob)                                   # canaries in the holes and after the end
    assert host_alltoallv(plan, send, recv, prob.counts, prob.sdispls, prob.rdispls, ts) == 0
    assert oracle.first_mismatch(recv, oracle.expected_recv(prob, send)) is None, args


def digits(d, r):
    out = []
    while d:
        out.append(d % r)
        d //= r
    return out


@settings(**COMMON)
@given(algo=st.sampled_from(BRUCK), P=st.integers(2, 20), r=st.integers(2, 21), b=st.integers(0, 3))
def test_bruck_blocks_hop_once_per_nonzero_digit(algo, P, r, b):
    plan = Plan(algo, P, r=r, b=b)
    if plan.err:
        return
    ops = plan.ops()
    r_eff = int(plan.spec["r"])                   # TuNA clamps the radix to the rank count
    paths = {}
    for o in sorted(ops, key=lambda o: int(o["key"])):
        paths.setdefault((int(o["origin"]), int(o["dest"])), []).append((int(o["src"]), int(o["dst"])))
    sign = None
    for (origin, dest), hops in paths.items():
        # the hops of one block form a chain origin -> ... -> dest
        assert hops[0][0] == origin and hops[-1][1] == dest
        for (s0, d0), (s1, d1) in zip(hops, hops[1:]):
            assert d0 == s1
        if origin == dest:
            assert hops == [(origin, origin)]
            continue
        fwd, bwd = (dest - origin) % P, (origin - dest) % P
        steps_fwd = sorted((d - s) % P for s, d in hops)
        steps_bwd = sorted((s - d) % P for s, d in hops)
        want_fwd = sorted(dg * r_eff ** x for x, dg in enumerate(digits(fwd, r_eff)) if dg)
        want_bwd = sorted(dg * r_eff ** x for x, dg in enumerate(digits(bwd, r_eff)) if dg)
        ok_fwd, ok_bwd = steps_fwd == want_fwd, steps_bwd == want_bwd
        assert ok_fwd or ok_bwd, (algo, P, r, origin, dest, hops)
        if fwd != bwd and ok_fwd != ok_bwd:       # the direction of travel is the same for every block of a plan
            this = "fwd" if ok_fwd else "bwd"
            sign = sign or this
            assert sign == this


@settings(**COMMON)
@given(args=plan_args())
def test_cells_written_once_before_they_are_read(args):
    plan = Plan(**args)
    if plan.err:
        return
    ops = plan.ops()
    written, read = {}, {}
    for i, o in enumerate(ops):
        if o["src_cell"] >= 0:
            k = (int(o["src"]), int(o["src_cell"]))
            assert k not in read
            read[k] = i
        if o["dst_cell"] >= 0:
            k = (int(o["dst"]), int(o["dst_cell"]))
            assert k not in written
            written[k] = i
            assert int(o["dst_cell"]) < plan.ncells
    assert set(read) <= set(written)
    for k, i in read.items():
        assert ops[written[k]]["key"] < ops[i]["key"]
    # every block reaches its destination once (a block sent in slices counts by its first slice)
    final = [o for o in ops[ops["dst_cell"] < 0] if ((int(o["flags"]) >> 2) & 127) == 0]
    P = args["P"]
    assert sorted((int(o["origin"]), int(o["dest"])) for o in final) == [(s, d) for s in range(P) for d in range(P)]
