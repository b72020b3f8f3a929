"""Pins the C oracle to the reference: every golden fixture in tests/golden was produced
by the unmodified naju_scan_reference (naju/scan.py:79-93 of the reference project)."""
import numpy as np
import pytest

import oracle
from conftest import golden_names, load_golden

GRADS = ("du", "dfl", "dil", "dB", "dC", "dD")


@pytest.mark.parametrize("precision", ["f32", "f64"])
@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_fixture(name, precision):
    d, ref = load_golden(name)
    args = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"])
    if "hT" in ref:
        y, hT = oracle.oracle_fwd(*args, h0=d["h0"], return_final_state=True, precision=precision)
        assert oracle.rel_l2(hT, ref["hT"]) < 2e-6
        g = oracle.oracle_bwd(*args, d["dy"], h0=d["h0"], dhT=d["dhT"], precision=precision)
        assert oracle.rel_l2(g["dh0"], ref["dh0"]) < 5e-6
    else:
        y = oracle.oracle_fwd(*args, precision=precision)
        g = oracle.oracle_bwd(*args, d["dy"], precision=precision)
    assert oracle.rel_l2(y, ref["y"]) < 2e-6
    for k in GRADS:
        assert oracle.rel_l2(g[k], ref[k]) < 5e-6, k


def test_step_equals_one_scan_iteration():
    d, ref = load_golden("step_B3_T1_D40_N16")
    y, st = oracle.oracle_step(d["h0"], d["u"][:, 0], d["fl"][:, 0], d["il"][:, 0],
                               d["Bm"][:, 0], d["Cm"][:, 0], d["Dskip"])
    assert oracle.rel_l2(y, ref["y"][:, 0]) < 2e-6
    assert oracle.rel_l2(st, ref["hT"]) < 2e-6


def test_composition_law():
    """Scanning [0,T) equals scanning [0,s) then [s,T) from the first part's final state
    (the identity naju/tests/test_affine_chunk.py:47-78 checks in torch)."""
    d = oracle.make_inputs(2, 80, 24, 16, seed=3)
    a = (d["u"], d["fl"], d["il"], d["Bm"], d["Cm"])
    y, hT = oracle.oracle_fwd(*a, d["Dskip"], return_final_state=True)
    s = 37
    y1, h1 = oracle.oracle_fwd(*(x[:, :s] for x in a), d["Dskip"], return_final_state=True)
    y2, h2 = oracle.oracle_fwd(*(x[:, s:] for x in a), d["Dskip"], h0=h1, return_final_state=True)
    assert np.abs(np.concatenate([y1, y2], 1) - y).max() < 1e-6
    assert np.abs(h2 - hT).max() < 1e-6


def test_empty_time_axis():
    d = oracle.make_inputs(1, 0, 8, 16, seed=1, with_h0=True)
    y, hT = oracle.oracle_fwd(d["u"], d["fl"], d["il"], d["Bm"], d["Cm"], d["Dskip"],
                              h0=d["h0"], return_final_state=True)
    assert y.shape == (1, 0, 8)
    assert np.array_equal(hT, d["h0"])
