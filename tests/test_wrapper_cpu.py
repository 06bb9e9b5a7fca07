"""Host logic of the op wrapper and the tuner, with the build and the kernels faked."""
import pytest
import torch

from fray_b200.jit_kernels import flashattn_cute as op
from fray_b200.jit_kernels import tuner as tuner_mod
from fray_b200.multi_gpu import shard_units


def test_cpu_tensors_are_refused():
    t = torch.zeros(1, 1, 128, 64, dtype=torch.half)
    with pytest.raises(AssertionError, match="no CPU path"):
        op.flash_attn_cute(t, t, t, t.clone())


def test_dtype_and_shape_contract():
    t = torch.zeros(1, 1, 128, 64, dtype=torch.float)
    with pytest.raises(AssertionError):
        op.flash_attn_cute(t, t, t, t.clone())
    a = torch.zeros(1, 1, 128, 64, dtype=torch.half)
    b = torch.zeros(1, 1, 256, 64, dtype=torch.half)
    with pytest.raises(AssertionError):
        op.flash_attn_cute(a, b, b, a.clone())


def test_arg_table_matches_template():
    names = [n for n, _ in op.arg_defs]
    assert names[:7] == ["Q", "K", "V", "O", "batch_size", "num_heads", "seq_len"]
    assert names[-3:] == ["causal", "scale", "stream"]
    for n in names:
        assert n in op.template
    for key in ("{KIND}", "{D}", "{BLOCK_N}", "{STAGES}"):
        assert key in op.template


def test_usable_strides():
    base = torch.zeros(2, 256, 4, 64, dtype=torch.half)
    assert op._usable_strides(base.transpose(1, 2))            # [B,S,H,D] viewed as [B,H,S,D]
    assert not op._usable_strides(base.transpose(2, 3))        # last dim not contiguous
    odd = torch.zeros(2, 4, 256, 68, dtype=torch.half)[..., :64]
    assert not op._usable_strides(odd)                         # row pitch 136 bytes: not a multiple of 16


def test_forced_space(monkeypatch):
    monkeypatch.setenv("FRAY_ATTN_FORCE", "KIND=0, BLOCK_N=64, STAGES=1")
    assert op.tuning_space(128) == ({"KIND": 0, "BLOCK_N": 64, "STAGES": 1},)
    monkeypatch.setenv("FRAY_ATTN_FORCE", "KIND=3,STAGES=6")
    assert op.tuning_space(128) == ({"KIND": 3, "BLOCK_N": 128, "STAGES": 6},)
    with pytest.raises(ValueError, match="head dim 128"):
        op.tuning_space(64)              # the paired kernel splits V into two 64-dim halves


def test_tuning_space_varies_tile_rows_stages_and_cta_pairing(monkeypatch):
    monkeypatch.delenv("FRAY_ATTN_FORCE", raising=False)
    for d in (64, 128):
        space = op.tuning_space(d)
        assert len({tuple(sorted(p.items())) for p in space}) == len(space)          # no duplicates
        assert {p["KIND"] for p in space} >= {op.KIND_SIMPLE, op.KIND_TWO_TILES, op.KIND_ALTERNATING}
        assert len({p["STAGES"] for p in space if p["KIND"] == op.KIND_TWO_TILES}) >= 2    # pipeline depth is searched
        assert {p["BLOCK_N"] for p in space} == {64, 128}
    assert op.KIND_PAIRED in {p["KIND"] for p in op.tuning_space(128)}               # 2-CTA MMA is a dimension at D = 128
    assert op.KIND_PAIRED not in {p["KIND"] for p in op.tuning_space(64)}


def test_prebuild_point_list_keeps_the_whole_space_when_a_point_is_forced(monkeypatch):
    monkeypatch.delenv("FRAY_ATTN_FORCE", raising=False)
    whole = op._space_points((64, 128), forced=False)
    monkeypatch.setenv("FRAY_ATTN_FORCE", "KIND=0,BLOCK_N=64,STAGES=1")
    assert op._space_points((64, 128), forced=False) == whole        # pruning keeps these
    assert len(op._space_points((64, 128), forced=True)) == 4        # 2 head dims x fp16/bf16
    assert op.os.environ["FRAY_ATTN_FORCE"] == "KIND=0,BLOCK_N=64,STAGES=1"


def test_status_of_a_process_that_launched_nothing():
    assert op.flash_attn_status() == (0, 0, 0, 0)


def test_fast_path_cache_is_bounded(monkeypatch):
    monkeypatch.setattr(op, "_fast_path", op.OrderedDict())
    for i in range(3 * op._FAST_PATH_ENTRIES):
        op._fast_path[i] = i
        while len(op._fast_path) > op._FAST_PATH_ENTRIES:
            op._fast_path.popitem(last=False)
    assert len(op._fast_path) == op._FAST_PATH_ENTRIES and (3 * op._FAST_PATH_ENTRIES - 1) in op._fast_path


def test_host_entry_refuses_pageable_and_mismatched_operands():
    t = torch.zeros(1, 2, 128, 64, dtype=torch.half)
    with pytest.raises(AssertionError, match="pinned"):
        op.flash_attn_cute_host(t, t, t, t.clone())


class FakeRuntime:
    def __init__(self, keys, rc=0, ms=1.0):
        self.keys, self.rc, self.ms, self.calls = keys, rc, ms, 0

    def __call__(self, *args):
        self.calls += 1
        return self.rc


def _fake_tuner(monkeypatch, table, tmp_path):
    monkeypatch.setenv("FRAY_CACHE_DIR", str(tmp_path))
    made = {}

    def fake_build(name, arg_defs, code):
        return made.setdefault(code, table[code])

    monkeypatch.setattr(tuner_mod, "build", fake_build)
    monkeypatch.setattr(tuner_mod, "generate", lambda inc, ad, body, epi="": body.strip())
    monkeypatch.setattr(tuner_mod.JITTuner, "time_candidate", staticmethod(lambda rt, args, launches=20: rt.ms))
    return tuner_mod.JITTuner()


def test_tuner_picks_fastest_legal_candidate_and_memoises(monkeypatch, tmp_path):
    table = {"k<1>": FakeRuntime(1, ms=3.0), "k<2>": FakeRuntime(2, rc=7, ms=0.1), "k<3>": FakeRuntime(3, ms=2.0)}
    t = _fake_tuner(monkeypatch, table, tmp_path)
    space = ({"T": 1}, {"T": 2}, {"T": 3})
    best = t.compile_and_tune("k", {"D": 64}, space, (), (), "k<{T}>", args=())
    assert best is table["k<3>"]                 # fastest among those whose launch returned 0
    assert table["k<2>"].calls == 1              # the illegal one was probed once and dropped
    assert t.compile_and_tune("k", {"D": 64}, space, (), (), "k<{T}>", args=()) is best
    # a second process (new tuner object) reuses the recorded winner without timing anything
    t2 = tuner_mod.JITTuner()
    monkeypatch.setattr(tuner_mod.JITTuner, "time_candidate",
                        staticmethod(lambda *a, **k: (_ for _ in ()).throw(AssertionError("timed again"))))
    assert t2.compile_and_tune("k", {"D": 64}, space, (), (), "k<{T}>", args=()) is best
    # a different workload class is tuned separately
    monkeypatch.setattr(tuner_mod.JITTuner, "time_candidate", staticmethod(lambda rt, args, launches=20: -rt.ms))
    assert t2.compile_and_tune("k", {"D": 128}, space, (), (), "k<{T}>", args=()) is table["k<1>"]


def test_tuner_fails_when_nothing_is_legal(monkeypatch, tmp_path):
    table = {"k<1>": FakeRuntime(1, rc=1), "k<2>": FakeRuntime(2, rc=1)}
    t = _fake_tuner(monkeypatch, table, tmp_path)
    with pytest.raises(AssertionError, match="Failed to tune"):
        t.compile_and_tune("k", {}, ({"T": 1}, {"T": 2}), (), (), "k<{T}>", args=())


@pytest.mark.parametrize("n,world", [(128, 1), (128, 8), (32, 8), (10, 4), (3, 8), (0, 2)])
def test_shard_units_partition(n, world):
    spans = [shard_units(n, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c and a <= b and c <= d
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1


def test_timeline_tool_parses_without_a_gpu():
    """The role-timeline tool imports nothing GPU-bound before it has parsed its arguments."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-m", "fray_b200.jit_kernels.timeline", "--help"], cwd=root,
                          capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr
    assert "--warm" in proc.stdout and "--row" in proc.stdout
