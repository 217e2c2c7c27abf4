"""``from mpi4py import MPI`` for the reference scripts: COMM_WORLD, Status, ANY_SOURCE."""
import datetime
import os
import pickle

import torch
import torch.distributed as dist

ANY_SOURCE = -1
ANY_TAG = -1


class Status:
    def __init__(self):
        self.source = -1
        self.tag = -1

    def Get_source(self):
        return self.source

    def Get_tag(self):
        return self.tag


class _Comm:
    def __init__(self):
        self._group = None

    def _g(self):
        if self._group is None:
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29533")
                dist.init_process_group("gloo", rank=int(os.environ.get("RANK", 0)),
                                        world_size=int(os.environ.get("WORLD_SIZE", 1)),
                                        timeout=datetime.timedelta(seconds=120))
                self._group = dist.group.WORLD
            elif "gloo" in str(dist.get_backend()):
                self._group = dist.group.WORLD
            else:
                self._group = dist.new_group(backend="gloo")
        return self._group

    def Get_rank(self):
        return dist.get_rank(self._g())

    def Get_size(self):
        return dist.get_world_size(self._g())

    def _send_bytes(self, payload: bytes, dest: int, tag: int):
        # MPI sends small messages eagerly (the reference relies on it: every rank sends to its neighbour
        # before anybody receives); a blocking gloo send would deadlock there, so post it and move on.
        g = self._g()
        head = torch.tensor([len(payload), tag], dtype=torch.int64, device="cpu")
        body = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
        self._inflight = [w for w in getattr(self, "_inflight", []) if not w[0].is_completed()]
        self._inflight.append((dist.isend(head, dest, group=g), head))
        self._inflight.append((dist.isend(body, dest, group=g), body))

    def send(self, obj, dest, tag=0):
        self._send_bytes(pickle.dumps(obj), dest, tag)

    def recv(self, source=ANY_SOURCE, tag=ANY_TAG, status=None):
        g = self._g()
        head = torch.zeros(2, dtype=torch.int64, device="cpu")
        if source == ANY_SOURCE:
            src = dist.recv(head, group=g)
        else:
            dist.recv(head, source, group=g)
            src = source
        buf = torch.empty(int(head[0]), dtype=torch.uint8, device="cpu")
        dist.recv(buf, src, group=g)
        if status is not None:
            status.source, status.tag = src, int(head[1])
        return pickle.loads(buf.numpy().tobytes())

    def bcast(self, obj, root=0):
        # the reference sets a CUDA default device; object collectives of gloo need host tensors
        box = [obj]
        dist.broadcast_object_list(box, src=root, group=self._g(), device=torch.device("cpu"))
        return box[0]

    def barrier(self):
        dist.barrier(group=self._g())

    Barrier = barrier


COMM_WORLD = _Comm()
