"""Host-side tile lists of the fused convolution launches: what every launch reads and writes, checked without a GPU.

The lists describe SO2_Convolution (src/fairchem/core/models/uma/nn/so2_layers.py:600-647: m=0 block, then one block
per |m| over [+m | -m]) followed by GateActivation (src/fairchem/core/models/uma/nn/activation.py:146-165: SiLU on the
l=0 row, sigmoid(gate of degree l) on the others) as 128-column output tiles."""

import pytest

from fairchem_b200 import backbone as B
from fairchem_b200 import ops

H = 128


def _shapes(lmax):
    ew = B.Edgewise(H, H, lmax, 2, [320, 128, 128])
    s1 = [tuple(w.shape) for w in B._conv_weights(ew.so2_conv_1)]
    s2 = [tuple(w.shape) for w in B._conv_weights(ew.so2_conv_2)]
    return s1, s2


def _tiles(flat):
    assert len(flat) % 9 == 0
    keys = ("a_col", "k", "w", "w_row", "out_col", "mode", "y_col", "gate_col", "flags")
    return [dict(zip(keys, flat[i:i + 9])) for i in range(0, len(flat), 9)]


@pytest.mark.parametrize("lmax", [2, 3, 4])
def test_every_output_column_is_written_once_and_operands_stay_in_range(lmax):
    s1, s2 = _shapes(lmax)
    lists = B.fused_conv_tile_lists(lmax, H, s1, s2)
    rows = len(B._row_degrees(lmax))
    gates = lmax * H
    widths = {  # (A columns, output columns written, m-block shapes, transposed)
        "fwd1": (sum(k for _, k in s1), rows * H, s1, False),
        "fwd1_keep": (sum(k for _, k in s1), rows * H, s1, False),
        "fwd2": (sum(k for _, k in s2), sum(n for n, _ in s2), s2, False),
        "bwd2": (sum(n for n, _ in s2), sum(k for _, k in s2), s2, True),
        "bwd1": (sum(n for n, _ in s1), sum(k for _, k in s1), s1, True),
    }
    for name, (a_cols, out_cols, shapes, transposed) in widths.items():
        tiles = _tiles(lists[name])
        assert len(tiles) <= ops.CONV_MAX_TILES
        gate_tiles = [t for t in tiles if name.startswith("fwd1") and t["mode"] == ops.CONV_PLAIN]
        assert len(gate_tiles) == (lmax if name.startswith("fwd1") else 0)
        written = sorted(t["out_col"] for t in tiles if t not in gate_tiles)
        # bwd2 writes grad y behind the gate columns, which the launch's last tiles of every degree fill
        base = gates if name == "bwd2" else 0
        assert written == [base + c for c in range(0, out_cols, 128)], name
        for t in tiles:
            n, k = shapes[t["w"]]
            w_rows, w_k = (k, n) if transposed else (n, k)
            assert t["k"] == w_k and t["k"] % 64 == 0
            assert 0 <= t["w_row"] and t["w_row"] + 128 <= w_rows
            assert 0 <= t["a_col"] and t["a_col"] + t["k"] <= a_cols
            assert t["a_col"] % 64 == 0 and t["out_col"] % 128 == 0


@pytest.mark.parametrize("lmax", [2, 4])
def test_gate_columns_follow_the_row_degree(lmax):
    s1, s2 = _shapes(lmax)
    lists = B.fused_conv_tile_lists(lmax, H, s1, s2)
    deg = B._row_degrees(lmax)
    gates = lmax * H
    for keep in (False, True):
        tiles = _tiles(lists["fwd1_keep" if keep else "fwd1"])
        # the gate columns are computed by the first lmax tiles, before any tile that reads them
        assert [t["mode"] for t in tiles[:lmax]] == [ops.CONV_PLAIN] * lmax
        assert [t["out_col"] for t in tiles[:lmax]] == [l * H for l in range(lmax)]
        for t in tiles[lmax:]:
            row = t["out_col"] // H
            assert t["y_col"] == gates + t["out_col"]
            assert bool(t["flags"] & ops.CONV_KEEP) == keep
            if deg[row] == 0:
                assert t["mode"] == ops.CONV_SILU
            else:
                assert t["mode"] == ops.CONV_GATED and t["gate_col"] == (deg[row] - 1) * H
    tiles = _tiles(lists["bwd2"])
    assert tiles[0]["mode"] == ops.CONV_SILU_BWD and tiles[0]["out_col"] == gates
    # the rows of a degree are consecutive, opened by FIRST and closed by LAST: the gate-gradient sum of a degree is
    # carried in registers between them and stored once
    rest = tiles[1:]
    seen = []
    i = 0
    while i < len(rest):
        l = rest[i]["gate_col"] // H + 1
        n_rows = deg.count(l)
        group = rest[i:i + n_rows]
        assert all(t["mode"] == ops.CONV_GATED_BWD and t["gate_col"] == (l - 1) * H for t in group)
        assert [deg[(t["out_col"] - gates) // H] for t in group] == [l] * n_rows
        assert [t["flags"] for t in group] == ([ops.CONV_FIRST | ops.CONV_LAST] if n_rows == 1 else
                                               [ops.CONV_FIRST] + [0] * (n_rows - 2) + [ops.CONV_LAST])
        seen.append(l)
        i += n_rows
    assert seen == list(range(1, lmax + 1))
    for name in ("fwd2", "bwd1"):
        assert all(t["mode"] == ops.CONV_PLAIN and t["flags"] == 0 for t in _tiles(lists[name]))
