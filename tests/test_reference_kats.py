"""The reference's closed-form known-answer samples: the oracle must reproduce them on
CPU (this pins the oracle and the graph interpreter), and the CUDA path must
reproduce them on the GPU."""
import pytest

from helpers import run_gpu
from kats import CASES
from oracle import fusilli_oracle as orc


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_reference_kat(name):
    g, ins, check = CASES[name]()
    assert check(orc.execute(g, ins)), name


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_gpu_reproduces_reference_kat(name):
    g, ins, check = CASES[name]()
    out = run_gpu(g, ins, repeat=2)  # the samples execute twice and re-check
    assert check(out), name
