"""The per-launch push policy of the fused collectives (how many CTAs push, what share of the tiles they keep)
on the shapes it was measured on; a stand-in answers the two library queries it makes."""
import pytest

from dizo_b200.parallel import fused


class _FakeLib:
    def dz_comm_gemm_grid(self, M, N, n_push, two):
        return 148

    def dz_comm_gemm_tiles(self, M, N, two):
        return ((M + 255) // 256) * ((N + 255) // 256)


@pytest.fixture
def plan(monkeypatch):
    monkeypatch.setattr(fused._lib, "lib", lambda: _FakeLib())
    fc = object.__new__(fused.FusedComm)
    fc.push_ctas, fc.push_share = 0, 0.0

    def run(world, M, N, K, nseg, rows, cols, two=1):
        fc.world = world
        d = fused._Desc()
        d.K, d.push_nseg, d.push_rows, d.push_cols = K, nseg, rows, cols
        return fc._push_plan(d, M, N, True, two)
    run.fc = fc
    return run


def test_two_ranks_every_cta_pushes(plan):
    assert plan(2, 8192, 10240, 5120, 1, 4096, 5120) == (148, 0)
    assert plan(2, 8192, 20480, 5120, 1, 10240, 5120) == (148, 0)


def test_four_ranks_sixteen_pushers_unless_the_transfer_outweighs_the_gemm(plan):
    assert plan(4, 8192, 9216, 9216, 1, 2048, 9216) == (16, -1)        # all-gather -> GEMM, 66B shapes
    assert plan(4, 8192, 20480, 5120, 1, 5120, 5120) == (16, -1)       # FSDP fc1, 13B shapes
    assert plan(4, 8192, 5120, 5120, 1, 2048, 5120) == (148, 0)        # all-gather -> GEMM, 13B shapes
    assert plan(4, 8192, 5120, 5120, 1, 5120, 5120) == (148, 0)        # FSDP: out_proj GEMM beside the fc1 push


def test_eight_ranks_balance_pushers_against_the_gemm(plan):
    assert plan(8, 8192, 20480, 5120, 1, 2560, 5120) == (16, -1)       # FSDP fc1: sixteen suffice
    n, join = plan(8, 8192, 5120, 5120, 1, 2560, 5120)                  # FSDP: out_proj GEMM beside the fc1 push
    assert 16 < n <= 64 and n % 2 == 0 and join == -1
    n2, _ = plan(8, 8192, 2560, 5120, 1, 1024, 5120)                    # all-gather -> GEMM, 13B shapes
    assert 16 < n2 <= 64


def test_overrides_and_push_only_launches(plan):
    assert plan(4, 0, 0, 5120, 1, 5120, 5120)[1] == 0                   # nothing to multiply: push only
    plan.fc.push_ctas, plan.fc.push_share = 32, 0.5
    n, join = plan(8, 8192, 20480, 5120, 1, 2560, 5120)
    assert n == 32 and 0 < join < 32 * 80
    plan.fc.push_ctas, plan.fc.push_share = 15, 0.0
    assert plan(8, 8192, 20480, 5120, 1, 2560, 5120, two=1) == (16, -1)  # CTA pairs push together
    assert plan(8, 8192, 20480, 5120, 1, 2560, 5120, two=0) == (15, -1)
