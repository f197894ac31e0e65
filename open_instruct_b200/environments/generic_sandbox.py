"""Sandboxed shell / editor environment with pluggable back ends.

Tools ``execute_bash`` (state - working directory and exported variables - persists between calls
through a wrapper script) and ``str_replace_editor`` (view / create / str_replace / insert), a
-0.05 penalty on errors and up to three reset attempts, as in the reference
(``open_instruct/environments/generic_sandbox.py:109-359``, back ends ``environments/backends.py:50-154``).
Back ends: ``LocalBackend`` (subprocess in a temporary directory) and ``DockerBackend`` (``docker run`` /
``docker exec``); tests substitute a mock back end.
"""

from __future__ import annotations

import abc
import os
import shlex
import shutil
import subprocess
import tempfile
from dataclasses import dataclass

from .base import RLEnvironment, StepResult, ToolCall

ERROR_PENALTY = -0.05


@dataclass
class ExecResult:
    stdout: str
    stderr: str = ""
    exit_code: int = 0


class SandboxBackend(abc.ABC):
    @abc.abstractmethod
    def start(self) -> None: ...

    @abc.abstractmethod
    def run(self, command: str, timeout: float = 30.0) -> ExecResult: ...

    @abc.abstractmethod
    def write_file(self, path: str, content: str) -> None: ...

    @abc.abstractmethod
    def read_file(self, path: str) -> str: ...

    def close(self) -> None:
        pass


class LocalBackend(SandboxBackend):
    def __init__(self):
        self.root = None

    def start(self):
        self.close()
        self.root = tempfile.mkdtemp(prefix="sandbox-")

    def _p(self, path):
        return path if os.path.isabs(path) and path.startswith(self.root) else os.path.join(self.root, path.lstrip("/"))

    def run(self, command, timeout=30.0):
        try:
            p = subprocess.run(["bash", "-c", command], cwd=self.root, capture_output=True, text=True, timeout=timeout)
            return ExecResult(p.stdout, p.stderr, p.returncode)
        except subprocess.TimeoutExpired:
            return ExecResult("", f"timed out after {timeout}s", 124)

    def write_file(self, path, content):
        full = self._p(path)
        os.makedirs(os.path.dirname(full) or ".", exist_ok=True)
        with open(full, "w") as fh:
            fh.write(content)

    def read_file(self, path):
        with open(self._p(path)) as fh:
            return fh.read()

    def close(self):
        if self.root and os.path.isdir(self.root):
            shutil.rmtree(self.root, ignore_errors=True)
        self.root = None


class DockerBackend(SandboxBackend):
    def __init__(self, image: str = "python:3.12-slim", mem_limit: str = "2g"):
        self.image, self.mem_limit, self.cid = image, mem_limit, None

    def start(self):
        self.close()
        p = subprocess.run(["docker", "run", "-d", "--rm", "--network", "none", "-m", self.mem_limit, self.image, "sleep", "infinity"],
                           capture_output=True, text=True, timeout=120)
        if p.returncode:
            raise RuntimeError(f"docker run failed: {p.stderr.strip()}")
        self.cid = p.stdout.strip()

    def run(self, command, timeout=30.0):
        try:
            p = subprocess.run(["docker", "exec", self.cid, "bash", "-c", command], capture_output=True, text=True, timeout=timeout)
            return ExecResult(p.stdout, p.stderr, p.returncode)
        except subprocess.TimeoutExpired:
            return ExecResult("", f"timed out after {timeout}s", 124)

    def write_file(self, path, content):
        subprocess.run(["docker", "exec", "-i", self.cid, "bash", "-c", f"mkdir -p $(dirname {shlex.quote(path)}) && cat > {shlex.quote(path)}"],
                       input=content, text=True, timeout=30, check=True)

    def read_file(self, path):
        return self.run(f"cat {shlex.quote(path)}").stdout

    def close(self):
        if self.cid:
            subprocess.run(["docker", "kill", self.cid], capture_output=True, timeout=30)
            self.cid = None


_STATE_FILE = ".sandbox_state"
_WRAPPER = ("touch {s}; source {s} 2>/dev/null; cd \"${{SANDBOX_CWD:-.}}\" 2>/dev/null; {cmd}\n__rc=$?\n"
            "{{ export -p; echo \"export SANDBOX_CWD=$(pwd)\"; }} > {s_abs}\nexit $__rc")


class GenericSandboxEnv(RLEnvironment):
    config_name = "generic_sandbox"

    def __init__(self, backend: SandboxBackend | str = "local", timeout: float = 30.0, max_output_chars: int = 8000, **backend_kw):
        self.backend = backend if isinstance(backend, SandboxBackend) else {"local": LocalBackend, "docker": DockerBackend}[backend](**backend_kw)
        self.timeout, self.max_output = timeout, max_output_chars

    @classmethod
    def get_tool_definitions(cls):
        return [
            {"type": "function", "function": {"name": "execute_bash", "description": "Run a bash command; cwd and exported variables persist.",
                                              "parameters": {"type": "object", "properties": {"command": {"type": "string"}}, "required": ["command"]}}},
            {"type": "function", "function": {"name": "str_replace_editor", "description": "View, create or edit files.",
                                              "parameters": {"type": "object", "properties": {
                                                  "command": {"type": "string", "enum": ["view", "create", "str_replace", "insert"]},
                                                  "path": {"type": "string"}, "file_text": {"type": "string"}, "old_str": {"type": "string"},
                                                  "new_str": {"type": "string"}, "insert_line": {"type": "integer"}},
                                                  "required": ["command", "path"]}}},
        ]

    def reset(self, setup_commands: list[str] | None = None, **_):
        last = None
        for _attempt in range(3):
            try:
                self.backend.start()
                for c in setup_commands or []:
                    self.backend.run(c, self.timeout)
                return StepResult("Sandbox ready.")
            except Exception as e:  # noqa: BLE001
                last = e
        raise RuntimeError(f"sandbox reset failed three times: {last}")

    def _clip(self, s: str) -> str:
        return s if len(s) <= self.max_output else s[: self.max_output] + f"\n... [{len(s) - self.max_output} characters truncated]"

    def _bash(self, command: str) -> StepResult:
        wrapped = _WRAPPER.format(s=_STATE_FILE, s_abs=f"$OLDPWD_ROOT/{_STATE_FILE}", cmd=command)
        res = self.backend.run("export OLDPWD_ROOT=$(pwd); " + wrapped, self.timeout)
        text = res.stdout + (("\n" + res.stderr) if res.stderr else "")
        return StepResult(self._clip(text.strip() or f"(exit code {res.exit_code})"), ERROR_PENALTY if res.exit_code else 0.0, False,
                          {"exit_code": res.exit_code})

    def _edit(self, a: dict) -> StepResult:
        cmd, path = a.get("command"), a.get("path", "")
        try:
            if cmd == "create":
                self.backend.write_file(path, a.get("file_text", ""))
                return StepResult(f"File created at {path}")
            text = self.backend.read_file(path)
            if cmd == "view":
                return StepResult(self._clip("\n".join(f"{i + 1:6d}\t{ln}" for i, ln in enumerate(text.splitlines()))))
            if cmd == "str_replace":
                old = a.get("old_str", "")
                n = text.count(old)
                if n != 1:
                    return StepResult(f"old_str must occur exactly once in {path} (found {n})", ERROR_PENALTY)
                self.backend.write_file(path, text.replace(old, a.get("new_str", "")))
                return StepResult(f"Edited {path}")
            if cmd == "insert":
                lines = text.splitlines(keepends=True)
                at = int(a.get("insert_line", len(lines)))
                new = a.get("new_str", "")
                lines[at:at] = [new if new.endswith("\n") else new + "\n"]
                self.backend.write_file(path, "".join(lines))
                return StepResult(f"Inserted into {path} at line {at}")
            return StepResult(f"unknown editor command {cmd}", ERROR_PENALTY)
        except Exception as e:  # noqa: BLE001
            return StepResult(f"{type(e).__name__}: {e}", ERROR_PENALTY)

    def step(self, call: ToolCall) -> StepResult:
        if call.name == "execute_bash":
            return self._bash(call.args.get("command", call.args.get("text", "")))
        if call.name == "str_replace_editor":
            return self._edit(call.args)
        return StepResult(f"unknown tool {call.name}", ERROR_PENALTY)

    def close(self):
        self.backend.close()
