"""Experiment tracking front-end (verl/utils/tracking.py:29-509): ``Tracking(project, experiment, backends,
config).log(data, step)``. Backends: console, file (JSONL), tensorboard, wandb, mlflow, swanlab, clearml,
trackio, vemlp_wandb; each third-party backend is imported lazily and reported clearly when absent.
"""

from __future__ import annotations

import dataclasses
import json
import os
from enum import Enum
from pathlib import Path
from typing import Any


def concat_dict_to_str(data: dict, step: int) -> str:
    parts = [f"step:{step}"]
    for k, v in data.items():
        if isinstance(v, (int, float)) or hasattr(v, "__float__"):
            try:
                parts.append(f"{k}:{float(v):.3f}")
            except (TypeError, ValueError):
                continue
    return " - ".join(parts)


class LocalLogger:
    def __init__(self, print_to_console: bool = True):
        self.print_to_console = print_to_console

    def flush(self):
        pass

    def log(self, data, step):
        if self.print_to_console:
            print(concat_dict_to_str(data, step), flush=True)


class FileLogger:
    """One JSON object per step in ``$VERL_FILE_LOGGER_PATH`` or ``$VERL_FILE_LOGGER_ROOT/<project>/<experiment>.jsonl``."""

    def __init__(self, project_name: str, experiment_name: str):
        path = os.getenv("VERL_FILE_LOGGER_PATH")
        if path is None:
            root = os.path.expanduser(os.getenv("VERL_FILE_LOGGER_ROOT", "."))
            d = os.path.join(root, project_name)
            os.makedirs(d, exist_ok=True)
            path = os.path.join(d, f"{experiment_name}.jsonl")
        else:
            os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        self.filepath = path
        self.fp = open(path, "w")
        print(f"Creating file logger at {path}")

    def log(self, data, step):
        self.fp.write(json.dumps({"step": step, "data": _jsonable(data)}) + "\n")

    def finish(self):
        self.fp.close()

    def flush(self):
        self.fp.flush()


def _jsonable(x):
    if isinstance(x, dict):
        return {str(k): _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    if isinstance(x, (str, int, float, bool)) or x is None:
        return x
    try:
        return float(x)
    except (TypeError, ValueError):
        return str(x)


class _TensorboardAdapter:
    def __init__(self, project_name, experiment_name):
        from torch.utils.tensorboard import SummaryWriter

        d = os.environ.get("TENSORBOARD_DIR", f"tensorboard_log/{project_name}/{experiment_name}")
        os.makedirs(d, exist_ok=True)
        print(f"Saving tensorboard log to {d}.")
        self.writer = SummaryWriter(d)

    def log(self, data, step):
        for k, v in data.items():
            try:
                self.writer.add_scalar(k, float(v), step)
            except (TypeError, ValueError):
                pass

    def finish(self):
        self.writer.close()


class _MlflowLoggingAdapter:
    def __init__(self):
        import mlflow

        self.mlflow = mlflow

    def log(self, data, step):
        import re

        self.mlflow.log_metrics({re.sub(r"[^a-zA-Z0-9_\-./ ]", "_", k).replace("@", "_at_"): float(v)
                                 for k, v in data.items() if _is_num(v)}, step=step)


def _is_num(v) -> bool:
    try:
        float(v)
        return True
    except (TypeError, ValueError):
        return False


def _flatten_dict(raw: dict, sep: str = "/") -> dict:
    out = {}

    def rec(prefix, node):
        for k, v in node.items():
            key = f"{prefix}{sep}{k}" if prefix else str(k)
            if isinstance(v, dict):
                rec(key, v)
            else:
                out[key] = v

    rec("", raw)
    return out


def _transform_params_to_json_serializable(x, convert_list_to_dict: bool):
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
        x = dataclasses.asdict(x)
    if isinstance(x, dict):
        return {k: _transform_params_to_json_serializable(v, convert_list_to_dict) for k, v in x.items()}
    if isinstance(x, list):
        if convert_list_to_dict:
            return {"list_len": len(x)} | {f"{i}": _transform_params_to_json_serializable(v, True) for i, v in enumerate(x)}
        return [_transform_params_to_json_serializable(v, False) for v in x]
    if isinstance(x, Path):
        return str(x)
    if isinstance(x, Enum):
        return x.value
    return x


class Tracking:
    supported_backend = ["wandb", "mlflow", "swanlab", "vemlp_wandb", "tensorboard", "console", "clearml", "trackio", "file"]

    def __init__(self, project_name, experiment_name, default_backend="console", config=None):
        if isinstance(default_backend, str):
            default_backend = [default_backend]
        for b in default_backend:
            assert b in self.supported_backend, f"{b} is not supported"
        self.logger: dict[str, Any] = {}
        cfg = _transform_params_to_json_serializable(config, convert_list_to_dict=False) if config is not None else None
        for b in default_backend:
            try:
                if b == "console":
                    self.logger[b] = LocalLogger(print_to_console=True)
                elif b == "file":
                    self.logger[b] = FileLogger(project_name, experiment_name)
                elif b == "tensorboard":
                    self.logger[b] = _TensorboardAdapter(project_name, experiment_name)
                elif b in ("wandb", "vemlp_wandb"):
                    import wandb

                    wandb.init(project=project_name, name=experiment_name, config=cfg)
                    self.logger[b] = wandb
                elif b == "mlflow":
                    import mlflow

                    mlflow.set_experiment(project_name)
                    mlflow.start_run(run_name=experiment_name)
                    if cfg:
                        mlflow.log_params(_flatten_dict(_transform_params_to_json_serializable(config, True)))
                    self.logger[b] = _MlflowLoggingAdapter()
                elif b == "swanlab":
                    import swanlab

                    swanlab.init(project=project_name, experiment_name=experiment_name, config=cfg)
                    self.logger[b] = swanlab
                elif b == "clearml":
                    import clearml

                    task = clearml.Task.init(project_name=project_name, task_name=experiment_name)
                    self.logger[b] = _ClearMLAdapter(task)
                elif b == "trackio":
                    import trackio

                    trackio.init(project=project_name, name=experiment_name, config=cfg)
                    self.logger[b] = trackio
            except ImportError as e:
                print(f"[tracking] backend '{b}' is not installed ({e}); it is skipped")

    def log(self, data, step, backend=None):
        for name, inst in self.logger.items():
            if backend is None or name in backend:
                if name in ("wandb", "vemlp_wandb", "swanlab", "trackio"):
                    inst.log(data=data, step=step)
                else:
                    inst.log(data, step)

    def __del__(self):
        for name, inst in getattr(self, "logger", {}).items():
            try:
                if name in ("wandb", "vemlp_wandb", "swanlab", "trackio"):
                    inst.finish()
                elif hasattr(inst, "finish"):
                    inst.finish()
            except Exception:
                pass


class _ClearMLAdapter:
    def __init__(self, task):
        self.task = task

    def log(self, data, step):
        lg = self.task.get_logger()
        for k, v in data.items():
            if _is_num(v):
                title, _, series = k.partition("/")
                lg.report_scalar(title=title, series=series or title, value=float(v), iteration=step)

    def finish(self):
        self.task.close()


class ValidationGenerationsLogger:
    """Logs (input, output, score) samples of validation to the active backends (table / text file)."""

    def __init__(self, project_name=None, experiment_name=None):
        self.project_name, self.experiment_name = project_name, experiment_name

    def log(self, loggers, samples, step):
        if "file" in loggers or "console" in loggers:
            d = os.path.join(os.path.expanduser(os.getenv("VERL_FILE_LOGGER_ROOT", ".")), self.project_name or "verl")
            os.makedirs(d, exist_ok=True)
            with open(os.path.join(d, f"{self.experiment_name or 'run'}_val_generations.jsonl"), "a") as f:
                for s in samples:
                    f.write(json.dumps({"step": step, "input": s[0], "output": s[1], "score": _jsonable(s[2])}) + "\n")
        if "wandb" in loggers:
            try:
                import wandb

                cols = ["step"] + sum([[f"input_{i+1}", f"output_{i+1}", f"score_{i+1}"] for i in range(len(samples))], [])
                row = [step] + [x for s in samples for x in s]
                wandb.log({"val/generations": wandb.Table(columns=cols, data=[row])}, step=step)
            except ImportError:
                pass
