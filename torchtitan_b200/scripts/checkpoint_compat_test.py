"""Checkpoint compatibility across two revisions of this code base.

    python -m torchtitan_b200.scripts.checkpoint_compat_test --old <git rev> [--new <git rev>] \
        --args "--module llama3 --config llama3_debugmodel" [--save-steps 5] [--total-steps 10]

The script checks out each revision into its own ``git worktree``, trains ``--save-steps`` steps
with the old revision and saves a checkpoint, resumes it with the new revision (default: the
working tree) up to ``--total-steps``, and compares the resumed losses with an uninterrupted run
of the new revision: they must be bit-identical (deterministic mode, same seed).  A difference
means the checkpoint format or the restored state (model, optimizer, LR schedule, dataloader)
changed between the revisions.  Parity: scripts/checkpoint_compat_test.py.
"""

from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys
import tempfile

_RUNNER = r"""
import json, sys
from torchtitan_b200.config import ConfigManager
argv, steps, out = json.loads(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
trainer = ConfigManager().parse_args(argv).build()
trainer.checkpointer.load()
losses = []
it = trainer.batch_generator(trainer.dataloader)
while trainer.step < steps:
    trainer.step += 1
    trainer.train_step(it)
    losses.append([trainer.step, float(trainer._last_loss)])
trainer.checkpointer.save(trainer.step, last_step=True)
trainer.close()
json.dump(losses, open(out, "w"))
"""


def _worktree(rev: str | None, root: str, tmp: str) -> str:
    if rev is None:
        return root
    path = os.path.join(tmp, "wt_" + rev.replace("/", "_"))
    subprocess.run(["git", "-C", root, "worktree", "add", "--detach", path, rev], check=True, capture_output=True)
    return path


def run(tree: str, arg_string: str, dump: str, steps: int, seed: int) -> list:
    argv = shlex.split(arg_string) + ["--debug.seed", str(seed), "--debug.deterministic", "--training.steps", str(10 ** 6),
                                      "--debug.no-enable_structured_logging", "--checkpoint.enable", "--checkpoint.interval",
                                      str(10 ** 6), "--dump_folder", dump]
    out = os.path.join(dump, f"losses_{steps}.json")
    os.makedirs(dump, exist_ok=True)
    env = dict(os.environ, PYTHONPATH=tree + os.pathsep + os.environ.get("PYTHONPATH", ""))
    subprocess.run([sys.executable, "-c", _RUNNER, json.dumps(argv), str(steps), out], check=True, cwd=tree, env=env)
    with open(out) as f:
        return json.load(f)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--old", required=True, help="git revision that writes the checkpoint")
    ap.add_argument("--new", default=None, help="git revision that resumes (default: the working tree)")
    ap.add_argument("--args", required=True, help="training arguments shared by all runs")
    ap.add_argument("--save-steps", type=int, default=5)
    ap.add_argument("--total-steps", type=int, default=10)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args(argv)
    root = subprocess.run(["git", "rev-parse", "--show-toplevel"], check=True, capture_output=True, text=True).stdout.strip()
    with tempfile.TemporaryDirectory() as tmp:
        old_tree, new_tree = _worktree(a.old, root, tmp), _worktree(a.new, root, tmp)
        try:
            resumed_dir, straight_dir = os.path.join(tmp, "resumed"), os.path.join(tmp, "straight")
            run(old_tree, a.args, resumed_dir, a.save_steps, a.seed)                    # old revision saves
            resumed = run(new_tree, a.args, resumed_dir, a.total_steps, a.seed)          # new revision resumes
            straight = run(new_tree, a.args, straight_dir, a.total_steps, a.seed)
        finally:
            for t in {old_tree, new_tree} - {root}:
                subprocess.run(["git", "-C", root, "worktree", "remove", "--force", t], capture_output=True)
    tail = [x for x in straight if x[0] > a.save_steps]
    ok = resumed == tail
    for (s, l1), (_, l2) in zip(resumed, tail):
        print(f"step {s}: resumed {l1!r}  uninterrupted {l2!r}{'' if l1 == l2 else '   <-- differs'}")
    print("checkpoint compatible: losses are bit-identical" if ok else "checkpoint INCOMPATIBLE")
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
