"""Environment backed by a task sandbox and a verifier (trl/experimental/harbor/_env.py: HarborEnv :37-206,
HarborBashEnv :209-231).

Per rollout: ``reset(task_dir)`` starts the task's sandbox and returns its instruction, tool methods execute inside the
sandbox, ``reward`` runs the task's verifier once, lazily, after the rollout.  Sandboxes: ``"local"`` runs commands in a
private copy of the task's ``environment/`` directory on this machine (no isolation beyond the working directory; for
trusted task suites and tests); any other ``environment_type`` is handed to the ``harbor`` package, which must be
installed."""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile

_NO_REWARD = object()


class _LocalSandbox:
    def __init__(self, task_dir: str):
        self.task_dir = task_dir
        self.workdir = tempfile.mkdtemp(prefix="harbor_local_")
        env_dir = os.path.join(task_dir, "environment")
        if os.path.isdir(env_dir):
            shutil.copytree(env_dir, self.workdir, dirs_exist_ok=True)

    def exec(self, command: str, timeout: int = 180) -> tuple[int, str]:
        try:
            r = subprocess.run(["bash", "-lc", command], cwd=self.workdir, capture_output=True, text=True, timeout=timeout)
            return r.returncode, (r.stdout + r.stderr)
        except subprocess.TimeoutExpired:
            return 124, f"command timed out after {timeout} s"

    def verify(self, timeout: int = 600) -> float:
        test = os.path.join(self.task_dir, "tests", "test.sh")
        if not os.path.exists(test):
            return 0.0
        rc, out = self.exec(f"bash {test!r}", timeout)
        reward_file = os.path.join(self.workdir, "reward.txt")
        if os.path.exists(reward_file):
            try:
                return float(open(reward_file).read().strip())
            except ValueError:
                pass
        return 1.0 if rc == 0 else 0.0

    def close(self):
        shutil.rmtree(self.workdir, ignore_errors=True)


class HarborEnv:
    PROMPT_SUFFIX: str = ""

    def __init__(self, environment_type: str = "docker"):
        self._environment_type = environment_type
        self._sandbox = None
        self._reward = _NO_REWARD

    def _open_sandbox(self, task_dir: str):
        if self._environment_type == "local":
            return _LocalSandbox(task_dir)
        try:
            import harbor  # noqa: F401
        except ImportError as e:
            raise ImportError(f"environment_type={self._environment_type!r} needs the `harbor` package; use "
                              "environment_type='local' for an unsandboxed working directory") from e
        raise NotImplementedError("remote Harbor sandboxes are reached through the harbor package's own client")

    def reset(self, task_dir: str | None = None, **kwargs) -> str:
        if task_dir is None:
            raise ValueError("HarborEnv.reset requires `task_dir` (provided by the dataset row).")
        self.close()
        self._sandbox = self._open_sandbox(task_dir)
        self._reward = _NO_REWARD
        with open(os.path.join(task_dir, "instruction.md")) as f:
            return f.read().strip() + self.PROMPT_SUFFIX

    def _exec(self, command: str, timeout: int = 180) -> str:
        rc, out = self._sandbox.exec(command, timeout)
        out = out if len(out) <= 8192 else out[:4096] + "\n...[truncated]...\n" + out[-4096:]
        return out if rc == 0 else f"{out}\n[exit code {rc}]"

    @property
    def reward(self) -> float:
        if self._reward is _NO_REWARD:
            self._reward = self._sandbox.verify() if self._sandbox is not None else 0.0
        return self._reward

    def close(self):
        if self._sandbox is not None:
            self._sandbox.close()
            self._sandbox = None


class HarborBashEnv(HarborEnv):
    PROMPT_SUFFIX = "\n\nYou can run shell commands with the `bash` tool. Finish when the task is solved."

    def bash(self, command: str) -> str:
        """Run a shell command in the task's sandbox.

        Args:
            command: The command line to execute.
        """
        return self._exec(command)


# built-in agent harnesses by name (``HarborSpec(agent="bash")``); extend with ``AGENTS["name"] = MyEnv``
AGENTS: dict[str, type[HarborEnv]] = {"bash": HarborBashEnv}
