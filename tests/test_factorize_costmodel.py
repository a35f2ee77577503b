"""Candidate enumeration and the original analytic cost model against golden data
captured from the reference tools (candidate lists, counts, chosen shape and cost for
N = 2..64 with chunk 100)."""
import math

import pytest

from allreduce_over_mpi_b200.parallel import planner as P

GOLDEN_CHOICE = """
2 1*2 .456 | 3 1*3 .549333 | 4 1*4 .596 | 5 1*5 .624 | 6 1*6 .642667 | 7 1*7 .656 | 8 1*8 .666 | 9 1*9 .673778
10 2*5 .688 | 11 1*11 .725091 | 12 2*6 .696 | 13 1*13 .772923 | 14 2*7 .701714 | 15 3*5 .709333 | 16 2*8 .706
17 1*17 .863059 | 18 2*9 .709333 | 19 1*19 .906526 | 20 4*5 .72 | 21 3*7 .716952 | 22 2*11 .754182 | 23 1*23 .991652
24 3*8 .719333 | 25 5*5 .7264 | 26 2*13 .797538 | 27 3*9 .721185 | 28 4*7 .724571 | 29 1*29 1.11669 | 30 5*6 .728
31 1*31 1.15794 | 32 4*8 .726 | 33 3*11 .763879 | 34 2*17 .881882 | 35 5*7 .729143 | 36 4*9 .727111 | 37 1*37 1.28086
38 2*19 .923368 | 39 3*13 .805744 | 40 5*8 .73 | 41 1*41 1.36234 | 42 6*7 .73219 | 43 1*43 1.40298 | 44 4*11 .768727
45 5*9 .730667 | 46 2*23 1.00557 | 47 1*47 1.48409 | 48 6*8 .732667 | 49 7*7 .734367 | 50 2*5*5 .7504 | 51 3*17 .888157
52 4*13 .809846 | 53 1*53 1.60543 | 54 6*9 .733037 | 55 5*11 .771636 | 56 7*8 .734571 | 57 3*19 .928982 | 58 2*29 1.12772
59 1*59 1.72651 | 60 2*5*6 .749333 | 61 1*61 1.76682 | 62 2*31 1.16826 | 63 7*9 .73473 | 64 8*8 .736
"""


def golden_rows():
    for cell in GOLDEN_CHOICE.replace("\n", "|").split("|"):
        cell = cell.strip()
        if cell:
            n, shape, cost = cell.split()
            yield int(n), shape, float(cost)


def test_prime_tools():
    assert P.prime_factors(840) == [2, 2, 2, 3, 5, 7]
    assert P.prime_factors(1) == [] and P.prime_factors(97) == [97]
    assert [n for n in range(1, 30) if P.is_prime(n)] == [2, 3, 5, 7, 11, 13, 17, 19, 23, 29]
    assert P.is_prime(1, loose=True) and not P.is_prime(1) and not P.is_prime(0, loose=True)


def test_candidates_golden_lists():
    assert P.candidate_shapes(8) == ["2*2*2", "2*4", "4*2", "1*8", "8*1"]
    assert P.candidate_shapes(12) == ["2*2*3", "2*3*2", "2*6", "3*2*2", "3*4", "4*3", "6*2", "1*12", "12*1"]
    assert P.candidate_shapes(7) == ["1*7", "7*1"]
    assert P.candidate_shapes(1) == [""] or P.candidate_shapes(1) == []
    assert P.candidate_shapes(0) == []
    for n, cnt in {2: 2, 4: 3, 6: 4, 8: 5, 12: 9, 16: 9, 18: 9, 20: 9}.items():
        assert len(P.candidate_shapes(n)) == cnt


def test_count_matches_enumeration():
    assert P.count_ordered_factorizations(0) == 0 and P.count_ordered_factorizations(1) == 1
    for n in range(2, 200):
        # the flat factorisation [n] is listed as the two sentinels 1*n and n*1
        assert len(P.candidate_shapes(n)) == P.count_ordered_factorizations(n) + 1


def test_legacy_enumerator_same_set():
    for n in list(range(2, 130)) + [256, 360, 512]:
        a, b = P.candidate_shapes(n), P.candidate_shapes(n, legacy=True)
        assert sorted(a) == sorted(b), n
        assert b[0] == f"1*{n}" and b[-1] == f"{n}*1"


def test_choose_width_readme_cases():
    # the hand-enumerated cases of the reference's cost-model notes for 7, 8, 9, 10 ranks
    assert set(P.choose_width(7)) == {"2*3+1", "3*2+1", "1*6+1", "6*1+1", "2*2*2-1", "2*4-1", "4*2-1", "1*8-1", "8*1-1"}
    c8 = P.choose_width(8)
    assert c8[:5] == ["2*2*2", "2*4", "4*2", "1*8", "8*1"] and "3*3-1" in c8 and "1*7+1" in c8
    c9 = set(P.choose_width(9))
    assert {"2*2*2+1", "2*4+1", "4*2+1", "3*3", "1*9", "9*1", "2*5-1", "5*2-1"} <= c9
    c10 = set(P.choose_width(10))
    assert {"3*3+1", "1*10", "10*1", "2*5", "5*2"} <= c10


def test_cost_v0_hand_check():
    # 1*8: 2 levels * 0.008 + (8 + 2*1 + 1) * 100/8 * 0.0004 + 7/8 * 100 * 0.0068
    assert P.cost_v0([1, 8], 8) == pytest.approx(0.016 + 0.055 + 0.595, abs=1e-12)
    # incast term: width 11 > 9 adds 100 * 2 * 0.0002
    assert P.cost_v0([1, 11], 11) - P.cost_v0([1, 11], 11, chunk=100) == 0
    assert P.cost_v0([11, 1], 11) > P.cost_v0([1, 11], 11)
    # arbitrary depth (the reference stops at 9 levels)
    assert math.isfinite(P.cost_v0([2] * 12, 4096))


@pytest.mark.parametrize("n,shape,cost", list(golden_rows()))
def test_choose_v0_golden(n, shape, cost):
    got_shape, got_cost, ncand = P.choose_v0(n)
    assert got_shape == shape
    assert float(f"{got_cost:.6g}") == cost  # the reference prints 6 significant digits
    assert ncand == len(P.candidate_shapes(n))


def test_v1_model_behaviour():
    k = P.CostParams(launch_us=4, sync_us=2, link_gbs=700, hbm_gbs=6000, nvls_gbs=0)
    big, small = 1 << 30, 4096
    flat, deep = P.Shape.parse("8"), P.Shape.parse("2*2*2")
    # every shape moves the same bytes per rank, so depth only adds rendezvous
    assert P.cost_v1(8, flat, big, k) < P.cost_v1(8, deep, big, k)
    assert P.cost_v1(8, deep, big, k) - P.cost_v1(8, flat, big, k) < 0.2 * P.cost_v1(8, flat, big, k)
    algo, shape, us = P.pick_algorithm(8, small, k)
    assert algo == "oneshot"
    algo, shape, us = P.pick_algorithm(8, big, k)
    assert algo == "staged" and str(shape) == "8"
    k.nvls_gbs = 1400
    assert P.pick_algorithm(8, big, k)[0] == "nvls"
    # bandwidth-optimal bound: >= 2*(N-1)/N * S / link
    assert P.cost_v1(8, flat, big, k) >= 2 * 7 / 8 * big / 700e3
    # round trip of the calibration table
    k2 = P.CostParams.from_json(k.to_json())
    assert k2 == k


def test_command_line_of_the_small_tools(capsys):
    """factor count, candidate printer, +1/-1 printer, model picks and schedule printer from one command line."""
    from allreduce_over_mpi_b200.parallel.__main__ import main
    assert main(["factor-count", "0", "1", "12", "64"]) == 0
    assert capsys.readouterr().out.split() == ["0", "1", "8", "32"]
    assert main(["candidates", "8"]) == 0
    assert capsys.readouterr().out.split() == ["2*2*2", "2*4", "4*2", "1*8", "8*1"]
    assert main(["choose-width", "7"]) == 0
    out = capsys.readouterr().out.split()
    assert "2*3+1" in out and "2*4-1" in out
    assert main(["choose", "10"]) == 0 and capsys.readouterr().out.startswith("2*5 0.688")
    assert main(["pick", "8", str(1 << 30)]) == 0 and capsys.readouterr().out.split()[0] in ("nvls", "staged", "push")
    assert main(["owners", "4", "1"]) == 0
    assert capsys.readouterr().out.splitlines() == ["block 0: rank 3", "block 1: rank 0", "block 2: rank 1", "block 3: rank 2"]
    assert main(["describe", "5", "2,2", "1"]) == 0
    out = capsys.readouterr().out
    assert "rank 4 of 5, shape 2*2+1, 4 stages" in out and out.count("stage 0 RS") == 5
    assert main(["describe", "7", "2,2", "3"]) == 1 and "invalid FT_TOPO" in capsys.readouterr().err
    assert main(["pick", "8"]) == 2
