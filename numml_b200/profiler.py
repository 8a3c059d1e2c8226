import time


class Profiler:
    """Nested wall-clock sections: ``with Profiler('label'): ...`` prints a tree of timings when
    the outermost section closes (reference ``numml/profiler.py:4-55``).  With ``sync=True`` the
    CUDA device is synchronised at both ends so that asynchronous kernels are charged to the
    section that launched them."""

    enabled = True
    current = None
    tab_width = 2
    sync = True

    def __init__(self, section_name):
        self.section_name = section_name
        self.children = []
        self.parent = None
        self.running_time = 0.0

    @staticmethod
    def _sync():
        if Profiler.sync:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()

    def __enter__(self):
        if not Profiler.enabled:
            return self
        self.parent = Profiler.current
        if self.parent is not None:
            self.parent.children.append(self)
        Profiler.current = self
        Profiler._sync()
        self.start_time = time.perf_counter()
        return self

    def report(self, level=0):
        print(' ' * (level * Profiler.tab_width) + f'[{self.section_name}] {self.running_time:.5f}s')
        for child in self.children:
            child.report(level + 1)

    def __exit__(self, exc_type, exc, tb):
        if not Profiler.enabled:
            return False
        Profiler._sync()
        self.running_time = time.perf_counter() - self.start_time
        Profiler.current = self.parent
        if self.parent is None and exc_type is None:
            self.report()
        return False
