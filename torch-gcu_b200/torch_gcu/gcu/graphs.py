"""Graph capture and replay for the gcu device (reference: torch_gcu/gcu/graphs.py:50-226).

    g = torch.gcu.GCUGraph()
    with torch.gcu.graph(g):          # runs the body once on a side stream, recording it
        static_out = step(static_in)
    static_in.copy_(new_input)
    g.replay()                        # one launch for the whole recorded sequence

Tensors created inside the capture live in a private pool of the allocator that exists
as long as the graph does; replays write the same addresses, so results are read from the
tensors the capture returned. Operators that synchronise with the host (item(), a copy to
the CPU) cannot be captured. Run the body eagerly at least once before capturing it, so
that one-time setup (kernel attributes, cached tables, communicators) is not recorded.
"""
import torch

import torch_gcu._C as _C


def is_current_stream_capturing() -> bool:
    return _C._gcu_isCurrentStreamCapturing()


class GCUGraph:
    def __init__(self):
        self._g = _C._GCUGraph()

    def capture_begin(self):
        self._g.capture_begin()

    def capture_end(self):
        self._g.capture_end()

    def replay(self):
        self._g.replay()

    def reset(self):
        self._g.reset()

    @property
    def captured(self) -> bool:
        return self._g.captured()

    @property
    def num_nodes(self) -> int:
        return self._g.num_nodes()


class graph:
    """Context manager: captures the body into `gcu_graph` on a side stream (`stream`, or a
    fresh one) that first waits for the work already queued on the current stream."""

    def __init__(self, gcu_graph: GCUGraph, stream=None):
        import torch_gcu.gcu as gcu
        self.g = gcu_graph
        self.stream = stream if stream is not None else gcu.Stream()
        self._ctx = None

    def __enter__(self):
        import torch_gcu.gcu as gcu
        gcu.synchronize()
        self.stream.wait_stream(gcu.current_stream())
        self._ctx = gcu.stream(self.stream)
        self._ctx.__enter__()
        self.g.capture_begin()
        return self.g

    def __exit__(self, exc_type, exc, tb):
        import torch_gcu.gcu as gcu
        try:
            if exc_type is None:
                self.g.capture_end()
            else:
                self.g.reset()
        finally:
            self._ctx.__exit__(exc_type, exc, tb)
        gcu.current_stream().wait_stream(self.stream)
        return False
