"""`python -m param_decomp_b200.experiments.lm.run_targeted <config.yaml> --data-root <dir>`

Targeted decomposition of an LM: a prompt-pool target stream plus a broad non-target stream per step.
Parity: param_decomp/experiments/lm/run_targeted.py:1-32.
"""

from __future__ import annotations

import argparse
import os
from pathlib import Path


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--data-root", "--data_root", type=Path, required=True)
    ap.add_argument("--run-id", "--run_id", type=str, default=None)
    ap.add_argument("--device", type=str, default=None)
    ap.add_argument("--local-device-count", "--local_device_count", type=int, default=None,
                    help="accepted for command lines written for the reference (one process per GPU here: the "
                         "launcher sets the process count); checked against LOCAL_WORLD_SIZE when both are known")
    ap.add_argument("--max-steps", "--max_steps", type=int, default=None)
    args = ap.parse_args(argv)
    local = os.environ.get("LOCAL_WORLD_SIZE")
    if args.local_device_count is not None and local is not None:
        assert int(local) == args.local_device_count, (
            f"--local-device-count {args.local_device_count}, but the launcher started {local} processes on this node")

    from param_decomp_b200.config.experiments import LMTargetedExperimentConfig

    cfg = LMTargetedExperimentConfig.from_file(args.config)
    for k, v in cfg.runtime.launch_env.rendered().items():
        os.environ.setdefault(k, v)

    from param_decomp_b200.experiments.lm.training import train_lm_targeted

    res = train_lm_targeted(cfg, args.data_root, run_id=args.run_id, device=args.device,
                            max_steps_this_entry=args.max_steps)
    if int(os.environ.get("RANK", "0")) == 0:
        print(f"finished at step {res.final_step}: {res.run_dir}")


if __name__ == "__main__":
    main()
