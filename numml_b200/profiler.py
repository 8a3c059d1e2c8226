"""Nested wall-clock sections.

    with Profiler('outer'):
        with Profiler('inner'):
            ...

prints, when the outermost section closes, one line per section indented by nesting depth
(same usage and output shape as the reference's ``numml/profiler.py:4-55``).  Unlike the reference,
the device is synchronised when a section opens and closes (``Profiler.sync``), so asynchronous
CUDA work is charged to the section that enqueued it, and every section is also an NVTX range
(``Profiler.nvtx``), so the same labels appear on the timeline of an attached GPU profiler.
"""
import time


class _Node:
    __slots__ = ("label", "parent", "children", "t0", "seconds")

    def __init__(self, label, parent):
        self.label, self.parent, self.children = label, parent, []
        self.t0 = self.seconds = 0.0
        if parent is not None:
            parent.children.append(self)

    def lines(self, depth, width):
        yield f"{' ' * (depth * width)}[{self.label}] {self.seconds:.5f}s"
        for child in self.children:
            yield from child.lines(depth + 1, width)


def _cuda_live():
    import torch
    return torch.cuda.is_available() and torch.cuda.is_initialized()


def _device_barrier():
    if _cuda_live():
        import torch
        torch.cuda.synchronize()


def _nvtx(push, label=None):
    if not _cuda_live():
        return False
    import torch
    if push:
        torch.cuda.nvtx.range_push(label)
    else:
        torch.cuda.nvtx.range_pop()
    return True


class Profiler:
    enabled = True      # set False to turn every section into a no-op
    sync = True         # synchronise the CUDA device at section boundaries
    nvtx = True         # open an NVTX range per section (a no-op unless a profiler is attached)
    tab_width = 2
    current = None      # innermost open section (a _Node), or None

    def __init__(self, section_name):
        self.section_name = section_name
        self._node = None
        self._ranged = False

    def __enter__(self):
        if Profiler.enabled:
            self._node = _Node(self.section_name, Profiler.current)
            Profiler.current = self._node
            if Profiler.sync:
                _device_barrier()
            self._ranged = Profiler.nvtx and _nvtx(True, self.section_name)
            self._node.t0 = time.perf_counter()
        return self

    def __exit__(self, exc_type, exc, tb):
        node = self._node
        if node is None:
            return False
        if Profiler.sync:
            _device_barrier()
        if self._ranged:
            _nvtx(False)
        node.seconds = time.perf_counter() - node.t0
        Profiler.current = node.parent
        if node.parent is None and exc_type is None:
            print("\n".join(node.lines(0, Profiler.tab_width)))
        return False

    @property
    def running_time(self):
        return self._node.seconds if self._node is not None else 0.0
