"""Data mixing and training phases (annealing): config rules, mixture sampler properties, phase transitions.

Mirrors the behaviours pinned by tests/unit/test_annealing.py and tests/unit/test_mixing.py of the reference.
"""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch
from torch.utils.data import Dataset

from kempnerforge_b200.config import load_config
from kempnerforge_b200.config.sections import DataConfig, DatasetSource, TrainingPhase
from kempnerforge_b200.data.dataset import MixtureDataset
from kempnerforge_b200.data.sampler import MixtureSampler
from kempnerforge_b200.training.trainer import Trainer, phase_weights


class _Const(Dataset):
    def __init__(self, n: int, tag: int) -> None:
        self.n, self.tag = n, tag

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i: int):
        if not 0 <= i < self.n:
            raise IndexError(i)
        return {"input_ids": torch.full((4,), self.tag), "labels": torch.full((4,), i)}


# --------------------------------------------------------------------------- config
def test_phase_defaults_and_fields():
    ph = TrainingPhase(start_step=10, dataset_weights={"a": 0.0, "b": 2.0}, lr_scale=0.5)
    assert (ph.start_step, ph.lr_scale, ph.dataset_weights["a"]) == (10, 0.5, 0.0)
    assert TrainingPhase().dataset_weights == {} and DataConfig().phases == []


@pytest.mark.parametrize("kwargs", [dict(start_step=-1), dict(lr_scale=0.0), dict(lr_scale=-1.0),
                                    dict(dataset_weights={"a": -0.1})])
def test_phase_rejects(kwargs):
    with pytest.raises(ValueError):
        TrainingPhase(**kwargs)


def test_phases_must_increase_strictly_and_exclude_the_shortcut():
    with pytest.raises(ValueError):
        DataConfig(phases=[TrainingPhase(start_step=10), TrainingPhase(start_step=5)])
    with pytest.raises(ValueError):
        DataConfig(phases=[TrainingPhase(start_step=10), TrainingPhase(start_step=10)])
    with pytest.raises(ValueError):
        DataConfig(phases=[TrainingPhase(start_step=10)], anneal_start_step=5, anneal_weights={"a": 1.0})
    with pytest.raises(ValueError):
        DataConfig(anneal_start_step=-1)


def test_anneal_shortcut_is_one_phase():
    dc = DataConfig(anneal_start_step=100, anneal_weights={"code": 3.0})
    (ph,) = dc.effective_phases()
    assert ph.start_step == 100 and ph.dataset_weights == {"code": 3.0} and ph.lr_scale == 1.0
    explicit = DataConfig(phases=[TrainingPhase(start_step=100, dataset_weights={"code": 3.0})]).effective_phases()
    assert explicit[0].start_step == ph.start_step and explicit[0].dataset_weights == ph.dataset_weights
    assert DataConfig(anneal_start_step=0, anneal_weights={"code": 3.0}).effective_phases() == []
    assert DataConfig(anneal_start_step=100).effective_phases() == []


def test_dataset_source_rules():
    assert DatasetSource(path="/x").weight == 1.0 and DatasetSource(hf_name="org/ds").name == ""
    with pytest.raises(ValueError):
        DatasetSource(path="/x", weight=0.0)
    with pytest.raises(ValueError):
        DataConfig(datasets=[DatasetSource(name="nothing")])
    with pytest.raises(ValueError):
        DataConfig(mix_temperature=0.0)
    assert DataConfig().datasets == [] and DataConfig().mix_temperature == 1.0


def test_phases_and_sources_load_from_toml(tmp_path):
    p = tmp_path / "c.toml"
    p.write_text(
        """
[data]
mix_temperature = 2.0
[[data.datasets]]
path = "/data/web"
weight = 3.0
name = "web"
[[data.datasets]]
hf_name = "org/code"
weight = 1.0
name = "code"
[[data.phases]]
start_step = 50
lr_scale = 0.5
dataset_weights = { web = 1.0, code = 4.0 }
[[data.phases]]
start_step = 80
"""
    )
    cfg = load_config(str(p))
    assert [s.name for s in cfg.data.datasets] == ["web", "code"] and cfg.data.datasets[1].hf_name == "org/code"
    assert cfg.data.mix_temperature == 2.0
    assert [ph.start_step for ph in cfg.data.phases] == [50, 80]
    assert cfg.data.phases[0].dataset_weights == {"web": 1.0, "code": 4.0} and cfg.data.phases[0].lr_scale == 0.5


def test_unknown_keys_inside_tables_are_rejected(tmp_path):
    for body in ('[[data.phases]]\nstart_step = 1\nbogus = 2\n', '[[data.datasets]]\npath = "/x"\nbogus = 2\n'):
        p = tmp_path / "bad.toml"
        p.write_text(body)
        with pytest.raises((ValueError, TypeError, KeyError)):
            load_config(str(p))


def test_anneal_shortcut_loads_from_toml(tmp_path):
    p = tmp_path / "c.toml"
    p.write_text('[data]\nanneal_start_step = 7\nanneal_weights = { a = 1.0, b = 0.0 }\n')
    cfg = load_config(str(p))
    assert cfg.data.anneal_start_step == 7 and cfg.data.anneal_weights == {"a": 1.0, "b": 0.0}
    assert cfg.data.effective_phases()[0].start_step == 7


# --------------------------------------------------------------------------- mixture dataset
def test_mixture_dataset_indexing():
    ds = MixtureDataset([_Const(5, 0), _Const(3, 1), _Const(4, 2)], ["a", "b", "c"])
    assert len(ds) == 12 and ds.cumulative_sizes == [0, 5, 8, 12] and ds.dataset_names == ["a", "b", "c"]
    for idx, (which, local) in {0: (0, 0), 4: (0, 4), 5: (1, 0), 7: (1, 2), 8: (2, 0), 11: (2, 3)}.items():
        s = ds[idx]
        assert int(s["dataset_idx"]) == which and int(s["input_ids"][0]) == which and int(s["labels"][0]) == local
    with pytest.raises(IndexError):
        ds[12]
    with pytest.raises(ValueError):
        MixtureDataset([], [])
    with pytest.raises(ValueError):
        MixtureDataset([_Const(1, 0)], ["a", "b"])
    assert ds.state_dict() == {}                      # sub-datasets without state contribute nothing

    class _Stateful(_Const):
        epoch = 0

        def state_dict(self):
            return {"epoch": self.epoch}

        def load_state_dict(self, state):
            self.epoch = state["epoch"]

    mixed = MixtureDataset([_Stateful(2, 0), _Const(2, 1), _Stateful(2, 2)], ["a", "b", "c"])
    mixed._datasets[2].epoch = 4
    state = mixed.state_dict()
    assert state == {"dataset_0": {"epoch": 0}, "dataset_2": {"epoch": 4}}
    fresh = MixtureDataset([_Stateful(2, 0), _Const(2, 1), _Stateful(2, 2)], ["a", "b", "c"])
    fresh.load_state_dict(state)
    assert fresh._datasets[2].epoch == 4
    fresh.load_state_dict({"datasets": [{"epoch": 9}, {}, {"epoch": 1}]})      # list form of older checkpoints
    assert fresh._datasets[0].epoch == 9 and fresh._datasets[2].epoch == 1


# --------------------------------------------------------------------------- mixture sampler
def _sampler(weights, sizes=(1000, 1000), **kw):
    cum = [0]
    for s in sizes:
        cum.append(cum[-1] + s)
    return MixtureSampler(cum, list(weights), kw.pop("num_replicas", 1), kw.pop("rank", 0), **kw), cum


def _shares(indices, cum):
    counts = [0] * (len(cum) - 1)
    for i in indices:
        for d in range(len(cum) - 1):
            if cum[d] <= i < cum[d + 1]:
                counts[d] += 1
    total = sum(counts)
    return [c / total for c in counts]


def test_sampler_total_and_proportions():
    s, cum = _sampler([3.0, 1.0])
    idx = list(s)
    assert len(idx) == len(s) == 2000 and all(0 <= i < 2000 for i in idx)
    a, b = _shares(idx, cum)
    assert abs(a - 0.75) < 0.01 and abs(b - 0.25) < 0.01


def test_sampler_oversamples_a_small_heavy_source():
    s, cum = _sampler([9.0, 1.0], sizes=(100, 900))
    idx = list(s)
    a, _ = _shares(idx, cum)
    assert abs(a - 0.9) < 0.01
    small = [i for i in idx if i < 100]
    assert len(small) > 100 and len(set(small)) == 100  # repeats, but every sample of the source is used


def test_sampler_is_deterministic_and_reshuffles_per_epoch():
    s1, _ = _sampler([1.0, 1.0], seed=3)
    s2, _ = _sampler([1.0, 1.0], seed=3)
    assert list(s1) == list(s2)
    first = list(s1)
    s1.set_epoch(1)
    assert list(s1) != first and sorted(list(s1)) != [] and len(list(s1)) == len(first)
    s3, _ = _sampler([1.0, 1.0], seed=4)
    assert list(s3) != first


def test_sampler_ranks_do_not_overlap_and_cover_their_share():
    per_rank = []
    for r in range(4):
        s, _ = _sampler([1.0, 1.0], num_replicas=4, rank=r, seed=1)
        per_rank.append(list(s))
    assert all(len(p) == 500 for p in per_rank)
    sets = [set(p) for p in per_rank]
    for i in range(4):
        for j in range(i + 1, 4):
            assert not (sets[i] & sets[j])
    assert len(set().union(*sets)) == 2000


def test_sampler_skip_ahead_and_state_round_trip():
    s, _ = _sampler([2.0, 1.0], seed=5)
    full = list(s)
    s.set_skip(37)
    assert list(s) == full[37:]
    assert list(s) == full  # the skip applies once
    s.set_epoch(2)
    state = s.state_dict()
    t, _ = _sampler([2.0, 1.0], seed=0)
    t.load_state_dict(state)
    assert list(t) == list(s)


@pytest.mark.parametrize("temperature,expect", [(1.0, 0.8), (100.0, 0.5), (0.25, 1.0)])
def test_sampler_temperature(temperature, expect):
    s, cum = _sampler([4.0, 1.0], temperature=temperature)
    a, _ = _shares(list(s), cum)
    assert abs(a - expect) < 0.02


@pytest.mark.parametrize("weights", [[], [0.0, 0.0], [-1.0, 2.0], [float("nan"), 1.0]])
def test_sampler_rejects_bad_weights(weights):
    with pytest.raises(ValueError):
        _sampler(weights)
    s, _ = _sampler([1.0, 1.0])
    with pytest.raises(ValueError):
        s.update_weights(weights)


def test_sampler_update_weights():
    s, cum = _sampler([1.0, 1.0])
    total = len(s)
    s.update_weights([1.0, 0.0])  # one zero beside a positive weight is fine
    idx = list(s)
    assert len(idx) == total and _shares(idx, cum) == [1.0, 0.0]
    s.update_weights([1.0, 3.0], temperature=1.0)
    assert abs(_shares(list(s), cum)[1] - 0.75) < 0.01
    with pytest.raises(ValueError):
        s.update_weights([1.0])


# --------------------------------------------------------------------------- phase transitions in the trainer
def _phase_host(phases, names=("web", "code"), weights=(3.0, 1.0), step=0):
    sampler, cum = _sampler(list(weights))
    loader = SimpleNamespace(sampler=sampler, dataset=SimpleNamespace(dataset_names=list(names)))
    cfg = SimpleNamespace(data=SimpleNamespace(datasets=[DatasetSource(path="/x", name=n, weight=w)
                                                         for n, w in zip(names, weights)], mix_temperature=1.0))
    host = SimpleNamespace(phases=phases, phase_idx=-1, step=step, dataloader=loader, config=cfg, _data_iter=object())
    return host, sampler, cum


def test_phase_weights_fall_back_to_configured_values():
    srcs = [DatasetSource(path="/a", name="web", weight=3.0), DatasetSource(path="/b", name="code", weight=1.0)]
    ph = TrainingPhase(start_step=1, dataset_weights={"code": 5.0})
    assert phase_weights(ph, ["web", "code"], srcs) == [3.0, 5.0]
    assert phase_weights(TrainingPhase(start_step=1, dataset_weights={"other": 9.0}), ["web", "code"], srcs) == [3.0, 1.0]


def test_phases_activate_in_order_at_their_steps():
    phases = [TrainingPhase(start_step=10, dataset_weights={"web": 1.0, "code": 1.0}, lr_scale=0.5),
              TrainingPhase(start_step=20, dataset_weights={"code": 9.0})]
    host, sampler, cum = _phase_host(phases)
    Trainer._maybe_advance_phase(host)
    assert host.phase_idx == -1 and host._data_iter is not None
    host.step = 10
    Trainer._maybe_advance_phase(host)
    assert host.phase_idx == 0 and host._data_iter is None
    assert abs(_shares(list(sampler), cum)[0] - 0.5) < 0.01
    host.step = 19
    Trainer._maybe_advance_phase(host)
    assert host.phase_idx == 0
    host.step = 20
    Trainer._maybe_advance_phase(host)
    assert host.phase_idx == 1
    assert abs(_shares(list(sampler), cum)[1] - 0.75) < 0.01  # web keeps its configured 3.0, code becomes 9.0


def test_resume_derives_phase_from_step_and_lr_scale_applies():
    phases = [TrainingPhase(start_step=10, lr_scale=0.5), TrainingPhase(start_step=20, lr_scale=0.1)]
    host, _, _ = _phase_host(phases, step=25)
    Trainer._maybe_advance_phase(host)
    assert host.phase_idx == 1
    host.optimizer = SimpleNamespace(param_groups=[{"lr": 1.0}, {"lr": 2.0}])
    Trainer._apply_phase_lr(host)
    assert [g["lr"] for g in host.optimizer.param_groups] == [0.1, 0.2]
