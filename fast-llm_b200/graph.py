"""Host-side mirror of the reference's ``Graph`` builder (``Graph::add`` /
``edge`` / ``freeze``, src/runtime/graph.cpp:19-93) and of ``Runtime::run`` for
the GPU side: a table of ``Task`` PODs with device pointers, handed to the
library as a plan (``fl_b200_plan_*``), which validates it with the reference's
freeze rules, merges row tiles and replays it as one CUDA graph."""
import ctypes as C

from . import capi


class Graph:
    def __init__(self, ctx):
        self.ctx = ctx
        self.lib = ctx.lib
        self._tasks = []
        self._keep = []      # device tensors holding parameter blocks
        self._plan = C.c_void_p()

    # -- Graph::add / edge --
    def add(self, kind, **fields):
        t = capi.Task()
        t.kind = kind
        t.nx = 1
        for k, v in fields.items():
            setattr(t, k, v)
        t.id = len(self._tasks)
        t.n_consumers = 0
        t.dep_init = 0
        self._tasks.append(t)
        return t.id

    def edge(self, producer, consumer):
        p = self._tasks[producer]
        if producer == consumer or consumer >= len(self._tasks):
            raise ValueError("bad edge")
        if p.n_consumers >= 6:
            raise ValueError("consumer fan-out exceeded")
        p.consumers[p.n_consumers] = consumer
        p.n_consumers += 1
        self._tasks[consumer].dep_init += 1

    def param_block(self, struct):
        """Copies a parameter POD (a ctypes Structure) to device memory; returns its device address."""
        import numpy as np
        import torch
        buf = torch.from_numpy(np.frombuffer(bytes(struct), dtype=np.uint8).copy()).cuda(self.ctx.device)
        self._keep.append(buf)
        return buf.data_ptr()

    # -- Graph::freeze + plan --
    def freeze(self):
        import torch
        torch.cuda.synchronize(self.ctx.device)   # the parameter blocks were uploaded on torch's stream
        arr = (capi.Task * len(self._tasks))(*self._tasks)
        capi._ck(self.lib.fl_b200_plan_create(self.ctx._h, arr, C.c_uint32(len(self._tasks)), C.byref(self._plan)))
        return self

    def run(self):
        capi._ck(self.lib.fl_b200_plan_run(self._plan))

    def info(self):
        a, b, c = C.c_uint32(), C.c_uint32(), C.c_uint32()
        capi._ck(self.lib.fl_b200_plan_info(self._plan, C.byref(a), C.byref(b), C.byref(c)))
        return dict(tasks=a.value, launches=b.value, merged_tiles=c.value)

    def close(self):
        if self._plan and self.ctx._h:
            self.lib.fl_b200_plan_destroy(self._plan)
        self._plan = C.c_void_p()
        self._keep = []
