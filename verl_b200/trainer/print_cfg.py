"""Print the fully composed trainer configuration (defaults lists, overrides and interpolations resolved); role of
the reference's ``scripts/print_cfg.py``.

    python -m verl_b200.trainer.print_cfg [ppo_trainer|sft_trainer] [key=value ...]
"""

from __future__ import annotations

import sys

import yaml

from ..utils.config import compose, to_container


def main(argv=None) -> str:
    args = list(sys.argv[1:] if argv is None else argv)
    name = args.pop(0) if args and "=" not in args[0] else "ppo_trainer"
    text = yaml.safe_dump(to_container(compose(name, args)), sort_keys=False, default_flow_style=False)
    print(text)
    return text


if __name__ == "__main__":
    main()
