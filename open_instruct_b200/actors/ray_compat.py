"""Actor runtime with the subset of the Ray API the GRPO system uses.

If ``ray`` is importable and ``OPEN_INSTRUCT_USE_RAY=1`` it is used unchanged.  Otherwise this module
provides the same calls on top of the standard library so the multi-process topology of the
reference (``open_instruct/grpo_fast.py:1245-1432``: learner actors, engine actors, a data-preparation
singleton, an actor manager, queues) runs without Ray:

    @remote                      class decorator             -> ActorClass
    ActorClass.options(num_gpus=1, name="x", env={...}).remote(*args)   -> ActorHandle (own OS process)
    handle.method.remote(*args)  -> ObjectRef (future)
    get(ref | [refs], timeout=)  / wait(refs, num_returns=, timeout=) / kill(handle) / get_actor(name)
    Queue(maxsize)               cross-process FIFO (an actor underneath), put/get/qsize/empty/put_nowait/get_nowait

Every actor process runs a small RPC server (``multiprocessing.connection.Listener`` on a unix
socket); a handle is just the socket address and is picklable, so handles can be passed to other
actors.  Calls to one actor run in a thread pool (``max_concurrency``), like Ray threaded actors.
GPUs are handed out by the driver through ``CUDA_VISIBLE_DEVICES``.
"""

from __future__ import annotations

import atexit
import concurrent.futures as cf
import multiprocessing as mp
import os
import pickle
import queue as _queue
import sys
import tempfile
import threading
import time
import traceback
import uuid
from multiprocessing.connection import Client, Listener

_USE_RAY = False
if os.environ.get("OPEN_INSTRUCT_USE_RAY") == "1":
    try:
        import ray as _ray  # noqa: F401

        _USE_RAY = True
    except ImportError:
        _USE_RAY = False

_AUTH = b"open-instruct-b200"
_named: dict[str, "ActorHandle"] = {}
_children: list[mp.Process] = []
_gpu_lock = threading.Lock()
_gpu_next = 0
_pool = cf.ThreadPoolExecutor(max_workers=64, thread_name_prefix="actor-call")


# ---------------------------------------------------------------------------------- wire format
# Control messages travel as plain pickles on the socket.  Bulk payloads - the packed batches the data-preparation producer
# hands to the learner ranks, weight vectors on CPU runs - would be copied through the socket in 64 KB pieces, so tensors
# and numpy arrays of a message that together exceed ``B200_ACTOR_SHM_MIN_BYTES`` (1 MiB) leave the pickle stream (protocol
# 5 out-of-band buffers) and go through ONE POSIX shared-memory segment: the sender writes them side by side, the socket
# carries the segment's name and the layout, the receiver copies them out and unlinks the segment.
_SHM_MAGIC = b"B2SHM1"
_SHM_MIN = int(os.environ.get("B200_ACTOR_SHM_MIN_BYTES", str(1 << 20)))
_SHM_MAX = int(os.environ.get("B200_ACTOR_SHM_MAX_BYTES", str(2 << 30)))   # larger payloads (whole models) keep to the socket


def _shm_has_room(nbytes: int) -> bool:
    """A segment is only created when /dev/shm can hold twice its size: running the tmpfs full ends in SIGBUS, not in an error."""
    try:
        st = os.statvfs("/dev/shm")
    except OSError:
        return False
    return st.f_bavail * st.f_frsize >= 2 * nbytes
_shm_sent: list[str] = []   # the last segments this process created: swept at exit in case a receiver died first


def _rebuild_tensor(buf, dtype_name: str, shape, pinned: bool):
    import numpy as np
    import torch

    a = np.frombuffer(buf, dtype=np.uint8)
    if not a.flags.writeable:
        a = a.copy()
    return torch.from_numpy(a).view(getattr(torch, dtype_name)).view(shape)


class _BulkPickler(pickle.Pickler):
    """Sends dense CPU tensors as out-of-band byte buffers (any dtype, bf16 included; non-contiguous ones are compacted)."""

    def reducer_override(self, obj):
        torch = sys.modules.get("torch")
        if torch is not None and isinstance(obj, torch.Tensor) and type(obj) is torch.Tensor and obj.device.type == "cpu" \
                and obj.layout == torch.strided and not obj.requires_grad and obj.numel() * obj.element_size() >= 4096:
            flat = obj.detach().contiguous().view(-1).view(torch.uint8)
            return _rebuild_tensor, (pickle.PickleBuffer(flat.numpy()), str(obj.dtype).replace("torch.", ""), tuple(obj.shape), False)
        return NotImplemented


def _dumps(obj) -> bytes:
    import io

    bufs: list[pickle.PickleBuffer] = []
    f = io.BytesIO()
    _BulkPickler(f, protocol=5, buffer_callback=bufs.append).dump(obj)
    views = [b.raw() for b in bufs]
    total = sum(v.nbytes for v in views)
    if total < _SHM_MIN or total > _SHM_MAX or not _shm_has_room(total):
        if not bufs:
            return f.getvalue()
        g = io.BytesIO()   # small (or far too large) payload: keep the buffers in band
        _BulkPickler(g, protocol=5).dump(obj)
        return g.getvalue()
    from multiprocessing import resource_tracker, shared_memory

    layout, off = [], 0
    for v in views:
        layout.append((off, v.nbytes))
        off += -(-v.nbytes // 64) * 64
    shm = shared_memory.SharedMemory(create=True, size=max(off, 1))
    try:
        for (o, n), v in zip(layout, views):
            shm.buf[o:o + n] = v
    finally:
        name = shm.name
        shm.close()
    try:  # the receiver unlinks; this process's tracker must not try again at exit
        resource_tracker.unregister("/" + name.lstrip("/"), "shared_memory")
    except Exception:  # noqa: BLE001
        pass
    _shm_sent.append(name)
    del _shm_sent[:-256]
    return _SHM_MAGIC + pickle.dumps((name, layout, f.getvalue()), protocol=5)


def _loads(raw: bytes):
    if not raw.startswith(_SHM_MAGIC):
        return pickle.loads(raw)
    from multiprocessing import shared_memory

    name, layout, data = pickle.loads(raw[len(_SHM_MAGIC):])
    shm = shared_memory.SharedMemory(name=name)
    try:
        bufs = [bytearray(shm.buf[o:o + n]) for o, n in layout]   # the one copy on this side; the segment goes away below
    finally:
        shm.close()
        try:
            shm.unlink()
        except FileNotFoundError:
            pass
    return pickle.loads(data, buffers=bufs)


def _sweep_segments() -> None:
    from multiprocessing import shared_memory

    for name in _shm_sent:
        try:
            seg = shared_memory.SharedMemory(name=name)
        except (FileNotFoundError, OSError):
            continue
        seg.close()
        try:
            seg.unlink()
        except FileNotFoundError:
            pass


atexit.register(_sweep_segments)


def _send(conn, obj) -> None:
    """Pickle by value (bulk buffers through shared memory, see above).  (``Connection.send`` would use multiprocessing's
    ForkingPickler, for which torch registers file-descriptor passing of tensors - a second channel between the processes
    whose lifetime rules we do not want for messages that are consumed once.)"""
    conn.send_bytes(_dumps(obj))


def _recv(conn):
    return _loads(conn.recv_bytes())


class ActorError(RuntimeError):
    """An exception raised inside an actor method, re-raised in the caller with the remote traceback."""


class ObjectRef:
    def __init__(self, fut: cf.Future):
        self._fut = fut

    def result(self, timeout=None):
        return self._fut.result(timeout)

    def done(self) -> bool:
        return self._fut.done()


def _serve(cls, args, kwargs, address, ready, max_concurrency, env):
    """Actor process main: build the object, answer calls until 'stop'."""
    os.environ.update(env)
    try:
        obj = cls(*args, **kwargs)
    except BaseException:  # noqa: BLE001
        ready.put(("error", traceback.format_exc()))
        return
    listener = Listener(address, family="AF_UNIX", authkey=_AUTH)
    ready.put(("ok", None))
    # one thread per client connection (connections are long-lived: every calling thread keeps its own); at most
    # ``max_concurrency`` method bodies run at a time
    running = threading.BoundedSemaphore(max(1, max_concurrency))
    stop = threading.Event()

    def bind_device():
        # CUDA's current device is a per-thread setting: give every serving thread the actor's GPU
        dev = getattr(obj, "device", None) or getattr(getattr(obj, "engine", None), "device", None)
        if dev is not None and str(dev).startswith("cuda"):
            import torch

            torch.cuda.set_device(torch.device(str(dev)))

    def handle(conn):
        try:
            bind_device()
            while not stop.is_set():
                try:
                    msg = _recv(conn)
                except (EOFError, OSError):
                    return
                if msg[0] == "stop":
                    stop.set()
                    _send(conn, ("ok", None))
                    return
                _, method, a, kw = msg
                try:
                    with running:
                        res = ("ok", getattr(obj, method)(*a, **kw))
                except BaseException as e:  # noqa: BLE001
                    res = ("error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
                try:
                    _send(conn, res)
                except Exception as e:  # noqa: BLE001 - unpicklable result
                    _send(conn, ("error", f"cannot send result of {method}: {e}"))
        finally:
            conn.close()

    listener._listener._socket.settimeout(0.2)
    while not stop.is_set():
        try:
            conn = listener.accept()
        except (OSError, _queue.Empty, TimeoutError):
            continue
        except Exception:  # noqa: BLE001
            continue
        threading.Thread(target=handle, args=(conn,), daemon=True, name="actor-conn").start()
    listener.close()
    if hasattr(obj, "shutdown"):
        try:
            obj.shutdown()
        except Exception:  # noqa: BLE001
            pass
    os._exit(0)


class _Method:
    def __init__(self, handle: "ActorHandle", name: str):
        self._h, self._name = handle, name

    def remote(self, *args, **kwargs) -> ObjectRef:
        return ObjectRef(_pool.submit(self._h._call, self._name, args, kwargs))


class ActorHandle:
    def __init__(self, address: str, pid: int | None = None, name: str | None = None):
        self._address, self._pid, self._name = address, pid, name
        self._local = threading.local()

    def __getstate__(self):
        return {"_address": self._address, "_pid": self._pid, "_name": self._name}

    def __setstate__(self, st):
        self.__dict__.update(st)
        self._local = threading.local()

    def _conn(self):
        c = getattr(self._local, "conn", None)
        if c is None:
            c = Client(self._address, family="AF_UNIX", authkey=_AUTH)
            self._local.conn = c
        return c

    def _call(self, method, args, kwargs):
        try:
            c = self._conn()
            _send(c, ("call", method, args, kwargs))
            status, val = _recv(c)
        except (EOFError, OSError, ConnectionError) as e:
            self._local.conn = None
            raise ActorError(f"actor {self._name or self._address} is not reachable: {e}") from e
        if status == "error":
            raise ActorError(val)
        return val

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return _Method(self, name)


class ActorClass:
    def __init__(self, cls, **opts):
        self._cls, self._opts = cls, opts

    def options(self, **opts) -> "ActorClass":
        return ActorClass(self._cls, **{**self._opts, **opts})

    def remote(self, *args, **kwargs) -> ActorHandle:
        global _gpu_next
        env = dict(self._opts.get("env", {}))
        n_gpu = self._opts.get("num_gpus", 0)
        if n_gpu and "CUDA_VISIBLE_DEVICES" not in env and "B200_GPU_IDS" not in env:
            with _gpu_lock:
                ids = list(range(_gpu_next, _gpu_next + int(max(1, n_gpu))))
                _gpu_next += int(max(1, n_gpu)) if n_gpu >= 1 else 0
            if self._opts.get("mask_gpus", False):
                visible = os.environ.get("CUDA_VISIBLE_DEVICES")
                pool = visible.split(",") if visible else None
                env["CUDA_VISIBLE_DEVICES"] = ",".join(pool[i] if pool else str(i) for i in ids)
            else:
                # every GPU stays visible (CUDA IPC and peer mappings need that); the actor picks its own
                env["B200_GPU_IDS"] = ",".join(str(i) for i in ids)
        address = os.path.join(tempfile.gettempdir(), f"oib200-{uuid.uuid4().hex[:12]}.sock")
        ctx = mp.get_context("spawn")
        ready = ctx.Queue()
        proc = ctx.Process(target=_serve, args=(self._cls, args, kwargs, address, ready, self._opts.get("max_concurrency", 8), env),
                           daemon=True)
        proc.start()
        # wait for the constructor, but notice a process that died in it (killed for memory, a crash in native code): such a
        # process never reports, and ranks that rendezvous with it would sit in their own timeouts
        deadline = time.time() + self._opts.get("init_timeout", 1200)
        while True:
            try:
                status, err = ready.get(timeout=0.5)
                break
            except _queue.Empty:
                if not proc.is_alive():
                    try:
                        status, err = ready.get(timeout=0.5)  # it may have reported just before exiting
                        break
                    except _queue.Empty:
                        raise ActorError(f"actor {self._cls.__name__} died while starting (exit code {proc.exitcode})") from None
                if time.time() > deadline:
                    proc.terminate()
                    raise ActorError(f"actor {self._cls.__name__} did not finish starting in time") from None
        if status != "ok":
            raise ActorError(f"actor {self._cls.__name__} failed to start:\n{err}")
        _children.append(proc)
        h = ActorHandle(address, proc.pid, self._opts.get("name"))
        if h._name:
            _named[h._name] = h
        return h


def remote(*args, **opts):
    """``@remote`` or ``@remote(num_gpus=1)`` on a class."""
    if len(args) == 1 and isinstance(args[0], type) and not opts:
        return ActorClass(args[0])
    return lambda cls: ActorClass(cls, **opts)


def get(refs, timeout: float | None = None):
    if isinstance(refs, ObjectRef):
        return refs.result(timeout)
    deadline = None if timeout is None else time.time() + timeout
    out = []
    for r in refs:
        out.append(r.result(None if deadline is None else max(0.0, deadline - time.time())))
    return out


def wait(refs, num_returns: int = 1, timeout: float | None = None):
    deadline = None if timeout is None else time.time() + timeout
    done, pending = [], list(refs)
    while len(done) < num_returns and pending:
        for r in list(pending):
            if r.done():
                done.append(r)
                pending.remove(r)
        if len(done) >= num_returns or (deadline is not None and time.time() >= deadline):
            break
        time.sleep(0.005)
    return done, pending


def get_actor(name: str) -> ActorHandle:
    if name not in _named:
        raise ValueError(f"no actor named {name}")
    return _named[name]


def kill(handle: ActorHandle) -> None:
    try:
        c = Client(handle._address, family="AF_UNIX", authkey=_AUTH)
        _send(c, ("stop",))
        if c.poll(5.0):
            _recv(c)
        c.close()
    except Exception:  # noqa: BLE001
        pass
    for p in list(_children):
        if p.pid == handle._pid:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
            _children.remove(p)
    try:
        os.unlink(handle._address)
    except OSError:
        pass
    if handle._name:
        _named.pop(handle._name, None)


def shutdown() -> None:
    """Stop every actor this process started."""
    global _gpu_next
    for p in list(_children):
        for h in [ActorHandle(a, p.pid) for a in ()]:
            pass
    for name, h in list(_named.items()):
        kill(h)
    for p in list(_children):
        if p.is_alive():
            p.terminate()
        p.join(timeout=2)
    _children.clear()
    _gpu_next = 0


class _QueueActor:
    def __init__(self, maxsize: int = 0):
        self.q = _queue.Queue(maxsize)

    def put(self, item, timeout=None):
        self.q.put(item, timeout=timeout)
        return True

    def put_nowait(self, item):
        self.q.put_nowait(item)
        return True

    def get(self, timeout=None):
        return self.q.get(timeout=timeout)

    def get_nowait(self):
        return self.q.get_nowait()

    def qsize(self):
        return self.q.qsize()


class Empty(Exception):
    pass


class Full(Exception):
    pass


class Queue:
    """FIFO shared between processes (cf. ``ray.util.queue.Queue``).  ``local=True`` keeps it in this
    process (threads only) - what the single-process GRPO mode and the tests use."""

    def __init__(self, maxsize: int = 0, local: bool = False):
        self.maxsize = maxsize
        self._local = _queue.Queue(maxsize) if local else None
        self._actor = None if local else ActorClass(_QueueActor, max_concurrency=32).remote(maxsize)

    def __getstate__(self):
        if self._local is not None:
            raise pickle.PicklingError("a local Queue cannot be sent to another process")
        return {"maxsize": self.maxsize, "_actor": self._actor, "_local": None}

    def __setstate__(self, st):
        self.__dict__.update(st)

    def put(self, item, block: bool = True, timeout: float | None = None):
        if self._local is not None:
            try:
                return self._local.put(item, block, timeout)
            except _queue.Full:
                raise Full from None
        try:
            get(self._actor.put.remote(item, timeout) if block else self._actor.put_nowait.remote(item))
        except ActorError as e:
            if "Full" in str(e):
                raise Full from None
            raise

    def put_nowait(self, item):
        return self.put(item, block=False)

    def get(self, block: bool = True, timeout: float | None = None):
        if self._local is not None:
            try:
                return self._local.get(block, timeout)
            except _queue.Empty:
                raise Empty from None
        try:
            return get(self._actor.get.remote(timeout) if block else self._actor.get_nowait.remote())
        except ActorError as e:
            if "Empty" in str(e):
                raise Empty from None
            raise

    def get_nowait(self):
        return self.get(block=False)

    def qsize(self) -> int:
        return self._local.qsize() if self._local is not None else get(self._actor.qsize.remote())

    def empty(self) -> bool:
        return self.qsize() == 0

    def shutdown(self):
        if self._actor is not None:
            kill(self._actor)
            self._actor = None
