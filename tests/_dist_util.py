"""Helpers for the multi-GPU child-process tests: a launcher that never leaves rank processes behind, and a
host-side deadline for the ranks themselves so that they leave between steps, with nothing in flight."""
import os
import signal
import subprocess
import sys
import threading
import time


def run_ranks(script: str, port: int, nproc: int = 2, timeout: float = 200.0, multimem: bool = False, extra_env=None):
    """Runs ``script`` on ``nproc`` ranks through torch.distributed.run in its own process group.  The ranks get a
    deadline 40 s shorter than the parent's, so a slow run ends by the ranks exiting on their own (arenas unmapped,
    communicators destroyed).  If the parent limit is hit all the same, the group gets SIGTERM, ten seconds, then
    SIGKILL.  NVLink multicast (NVLS / multimem) stays off unless a test asks for it: a rank that dies while bound
    to a multicast object can fault its peers."""
    env = dict(os.environ)
    env["TRL_B200_TEST_DEADLINE_S"] = str(max(20.0, timeout - 40.0))
    env.setdefault("NCCL_NVLS_ENABLE", "1" if multimem else "0")
    env["TRL_B200_MULTIMEM"] = "1" if multimem else "0"
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), script]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, start_new_session=True)
    try:
        out, err = p.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGTERM)
        try:
            out, err = p.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            os.killpg(p.pid, signal.SIGKILL)
            out, err = p.communicate()
        return -9, out, err + "\n[parent] time limit reached"
    return p.returncode, out, err


class Deadline:
    """Started by a rank at set-up; ``check()`` between steps raises SystemExit once the limit has passed."""

    def __init__(self, seconds: float | None = None):
        self.limit = float(os.environ.get("TRL_B200_TEST_DEADLINE_S", "0") or 0) if seconds is None else seconds
        self.expired = threading.Event()
        self.t0 = time.monotonic()
        if self.limit > 0:
            t = threading.Timer(self.limit, self.expired.set)
            t.daemon = True
            t.start()

    def check(self, where: str = ""):
        if self.expired.is_set():
            print(f"[rank {os.environ.get('RANK', '?')}] test deadline of {self.limit:.0f}s passed {where}; leaving", flush=True)
            try:
                import torch.distributed as td

                if td.is_initialized():
                    td.destroy_process_group()
            finally:
                raise SystemExit(3)


def greedy_gaps(model, prompt, tokens):
    """For a greedy completion ``tokens`` of ``prompt``: at every step, how far (in logit units, fp32 oracle forward of
    the same weights) the chosen token lies below the best one.  Greedy decoding of a tiny random model sits on
    near-ties, so two correct engines may pick different tokens; both must stay within rounding of the maximum."""
    import copy

    import torch

    m32 = copy.deepcopy(model).float().cpu()  # the plain fp32 path of the model
    ids = torch.tensor([list(prompt) + list(tokens)])
    with torch.no_grad():
        logits = m32(input_ids=ids).logits[0].float()
    steps = logits[len(prompt) - 1:len(prompt) - 1 + len(tokens)]
    chosen = steps.gather(1, torch.tensor(list(tokens))[:, None])[:, 0]
    return (steps.max(dim=1).values - chosen).tolist()
