"""IQ lattice tables built by the library (host code, no GPU needed) against the digests of the tables the
reference ships in seedpack/ggml/iqtables.npz (grids, maps and neighbour lists of iq2_data[0..3] and
iq3_data[0..1], as built by iq2xs_init_impl / iq3xs_init_impl).  tests/golden/make_table_digests.py wrote
the digests from that file."""
import hashlib
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_tables_match_reference_digests():
    from seedpack_b200 import tables
    want = json.load(open(os.path.join(HERE, "golden", "iq_table_digests.json")))
    for which in range(6):
        for what, kind in enumerate(("grid", "map", "nb")):
            a = tables.host(which, what)
            key = f"{which}_{kind}"
            assert a.size == want[key]["n"], key
            assert hashlib.sha256(a.tobytes()).hexdigest() == want[key]["sha256"], key
