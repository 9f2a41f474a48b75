"""Skip generation by replaying dumped rollouts (role of verl/utils/rollout_skip.py:19-120).

``RolloutSkip(config, rollout_wg).wrap_generate_sequences()`` replaces the worker group's ``generate_sequences``:
the first ``config.actor_rollout_ref.rollout.skip_rollout`` run stores every generated batch under
``skip_dump_dir`` (keyed by experiment, batch shape and step), later runs load them instead of generating, which
makes trainer-side debugging independent of the rollout engine.
"""

from __future__ import annotations

import os
from pathlib import Path

from ..protocol import DataProto


class RolloutSkip:
    def __init__(self, config, rollout_wg):
        rc = config.actor_rollout_ref.rollout
        self.rollout_wg = rollout_wg
        self.exp = f"{config.trainer.project_name}_{config.trainer.experiment_name}"
        self.n = int(rc.get("n", 1))
        self.gbs = int(config.data.get("gen_batch_size") or config.data.train_batch_size)
        self.prompt_length, self.response_length = int(config.data.max_prompt_length), int(config.data.max_response_length)
        self.dump_dir = Path(os.path.expanduser(str(rc.get("skip_dump_dir", "/tmp/rollout_dump"))))
        self.step = 0
        self._wrapped = False

    @property
    def curr_path_dump(self) -> Path:
        return self.dump_dir / f"{self.exp}_GBS{self.gbs}__N{self.n}__in{self.prompt_length}__out{self.response_length}" / f"step_{self.step}.pt"

    def try_load(self):
        p = self.curr_path_dump
        if not p.exists():
            return None
        try:
            return DataProto.load_from_disk(str(p))
        except Exception as e:  # a corrupt dump falls back to generating
            print(f"[RolloutSkip] failed to load {p}: {e}")
            return None

    def dump(self, out: DataProto) -> None:
        p = self.curr_path_dump
        p.parent.mkdir(parents=True, exist_ok=True)
        out.save_to_disk(str(p))

    def wrap_generate_sequences(self):
        if self._wrapped:
            return
        inner = self.rollout_wg.generate_sequences

        def generate_sequences(batch: DataProto, **kw) -> DataProto:
            self.step += 1
            cached = self.try_load()
            if cached is not None and len(cached) == len(batch) * (self.n if len(cached) != len(batch) else 1):
                return cached
            out = inner(batch, **kw)
            self.dump(out)
            return out

        self.rollout_wg.generate_sequences = generate_sequences
        self._wrapped = True
