"""Job-level observability outside the metric stream: alerts, progress lines, run tags, disk warnings.

Counterparts of the reference's helpers (``open_instruct/utils.py``: ``send_slack_message`` ``:2679-2699``,
``maybe_update_beaker_description`` ``:1106-1193`` with ``format_eta`` ``:1091-1103``, ``get_wandb_tags`` ``:767-784``,
``warn_if_low_disk_space`` ``:106-139``).  Everything here degrades to a log line when its service is not configured: no
webhook URL, no scheduler client, no network.  The scheduler integration goes through a small ``DescriptionSink`` interface
(a Beaker client is one implementation, picked up when ``beaker`` is importable and ``BEAKER_WORKLOAD_ID`` is set), so the
progress text is testable without any service.
"""

from __future__ import annotations

import logging
import os
import shutil
import subprocess
import time

logger = logging.getLogger(__name__)
DISK_USAGE_WARNING_THRESHOLD = 0.85
CLOUD_PATH_PREFIXES = ("gs://", "s3://", "az://", "hdfs://", "/filestore")


def format_eta(seconds: float) -> str:
    s = int(seconds)
    d, h, m = s // 86400, (s % 86400) // 3600, (s % 3600) // 60
    return f"{d}d {h}h {m}m" if d else (f"{h}h {m}m" if h else f"{m}m")


def progress_text(current_step: int, total_steps: int, elapsed_s: float) -> str:
    """``[12.5% complete (step 5/40), eta 1h 3m]`` / ``finished in ...`` / ``eta calculating...`` at step 0."""
    pct = 100.0 * current_step / max(total_steps, 1)
    if current_step >= total_steps:
        label, t = "finished in", format_eta(elapsed_s)
    elif current_step > 0:
        label, t = "eta", format_eta(elapsed_s / current_step * (total_steps - current_step))
    else:
        label, t = "eta", "calculating..."
    return f"[{pct:.1f}% complete (step {current_step}/{total_steps}), {label} {t}]"


class DescriptionSink:
    """Where a one-line job description lives (a scheduler's experiment page)."""

    def get(self) -> str:
        raise NotImplementedError

    def set(self, text: str) -> None:
        raise NotImplementedError

    def url(self) -> str | None:
        return None


class BeakerDescriptionSink(DescriptionSink):
    def __init__(self):
        import beaker  # noqa: F401 - only where the scheduler's client is installed

        self._client = beaker.Beaker.from_env()
        self._workload = self._client.workload.get(os.environ["BEAKER_WORKLOAD_ID"])

    def get(self) -> str:
        return self._client.experiment.get_spec(self._workload).description or ""

    def set(self, text: str) -> None:
        self._client.workload.update(self._workload, description=text)

    def url(self) -> str | None:
        try:
            return self._client.experiment.url(self._workload.experiment)
        except Exception:  # noqa: BLE001
            return None


def default_sink() -> DescriptionSink | None:
    if not os.environ.get("BEAKER_WORKLOAD_ID"):
        return None
    try:
        return BeakerDescriptionSink()
    except Exception as e:  # noqa: BLE001 - client missing or misconfigured: progress lines are optional
        logger.warning("no scheduler description sink: %s", e)
        return None


class ProgressReporter:
    """Keeps the job description current: ``<original text> git_commit: ... git_branch: ... [wandb url] [progress]``.  The
    original text is read once (anything after an earlier ``git_commit:`` is dropped, so restarts do not pile up)."""

    def __init__(self, total_steps: int, sink: DescriptionSink | None = None, wandb_url: str | None = None):
        self.total_steps, self.sink, self.wandb_url = total_steps, sink if sink is not None else default_sink(), wandb_url
        self.start = time.perf_counter()
        self._original: str | None = None

    def update(self, current_step: int | None = None) -> str | None:
        if self.sink is None:
            return None
        try:
            if self._original is None:
                self._original = self.sink.get().split("git_commit:")[0].strip()
            parts = [self._original, f"git_commit: {os.environ.get('GIT_COMMIT', 'unknown')}", f"git_branch: {os.environ.get('GIT_BRANCH', 'unknown')}"]
            if self.wandb_url:
                parts.append(self.wandb_url)
            if current_step is not None:
                parts.append(progress_text(current_step, self.total_steps, time.perf_counter() - self.start))
            text = " ".join(p for p in parts if p)
            self.sink.set(text)
            return text
        except Exception as e:  # noqa: BLE001 - a scheduler hiccup must not stop training
            logger.warning("could not update the job description: %s", e)
            return None


def send_slack_message(message: str, sink: DescriptionSink | None = None, post=None) -> bool:
    """POST ``{"text": message}`` to ``$SLACK_WEBHOOK_URL``; True when the webhook accepted it.  ``post`` replaces
    ``requests.post`` (tests)."""
    url = os.environ.get("SLACK_WEBHOOK_URL")
    if not url:
        logger.warning("SLACK_WEBHOOK_URL environment variable not set. Skipping Slack alert.")
        return False
    job = sink.url() if sink is not None else None
    payload = {"text": message + (f" Check it out: {job}" if job else "")}
    try:
        if post is None:
            import requests

            post = requests.post
        r = post(url, json=payload, timeout=10)
        if not getattr(r, "ok", False):
            logger.warning("Failed to send Slack alert with status %s: %s", getattr(r, "status_code", "?"), getattr(r, "text", ""))
            return False
        return True
    except Exception as exc:  # noqa: BLE001 - no network here
        logger.warning("Failed to send Slack alert due to network error: %s", exc)
        return False


def alert_on_failure(fn):
    """Decorator for entry points: a Slack alert with the exception's type and message when ``send_slack_alerts`` is on."""
    import functools

    @functools.wraps(fn)
    def wrapped(args, *a, **kw):
        try:
            return fn(args, *a, **kw)
        except Exception as e:
            if getattr(args, "send_slack_alerts", False):
                send_slack_message(f"<!here> A training job died: {type(e).__name__}: {e}")
            raise

    return wrapped


def warn_if_low_disk_space(path: str, threshold: float = DISK_USAGE_WARNING_THRESHOLD, send_slack_alerts: bool = False) -> str | None:
    """Warn when the filesystem holding ``path`` is fuller than ``threshold`` (checkpoints may fail); cloud paths are skipped."""
    if path.startswith(CLOUD_PATH_PREFIXES):
        return None
    probe = path
    while probe and not os.path.exists(probe):
        probe = os.path.dirname(probe.rstrip("/"))
    try:
        usage = shutil.disk_usage(probe or "/")
    except OSError as e:
        logger.warning("Skipping disk usage check for %s, encountered OS error: %s", path, e)
        return None
    if usage.total == 0 or usage.used / usage.total < threshold:
        return None
    msg = (f"Disk usage near capacity for {path}: {100 * usage.used / usage.total:.1f}% used ({usage.free / 2**30:.1f} GiB free of "
           f"{usage.total / 2**30:.1f} GiB). Checkpointing may fail.")
    logger.warning(msg)
    if send_slack_alerts:
        send_slack_message(msg)
    return msg


def get_git_commit() -> str:
    if os.environ.get("GIT_COMMIT"):
        return os.environ["GIT_COMMIT"]
    try:
        return subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5, check=True).stdout.strip() or "unknown"
    except Exception:  # noqa: BLE001
        return "unknown"


def get_wandb_tags() -> list[str]:
    """``$WANDB_TAGS`` plus ``commit: <sha>`` and ``branch: <name>`` (each at most 64 characters).  The reference also asks
    GitHub for the pull-request number of the commit; there is no network here, so that tag only appears when ``$GIT_PR`` is
    set by the launcher."""
    tags = [t for t in os.environ.get("WANDB_TAGS", "").split(",") if t]
    commit = get_git_commit()
    if commit != "unknown":
        tags.append(f"commit: {commit}")
    if os.environ.get("GIT_PR"):
        tags.append(f"pr: {os.environ['GIT_PR']}")
    if os.environ.get("GIT_BRANCH"):
        tags.append(f"branch: {os.environ['GIT_BRANCH']}")
    return [t[:64] for t in tags]
