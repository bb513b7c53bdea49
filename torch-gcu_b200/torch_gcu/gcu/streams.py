"""Stream and Event of the gcu backend (reference: torch_gcu/gcu/streams.py:13-237).
Both ride on PyTorch's device-generic torch.Stream / torch.Event, which call the
registered device guard; only the raw-handle accessors are backend specific."""
import torch

from torch_gcu import _C


class Stream(torch.Stream):
    """A stream of a gcu device. `Stream(device=None, priority=0)` takes one from the
    device's pool (priority -1: the high-priority pool)."""

    def __new__(cls, device=None, priority=0, **kwargs):
        if "stream_id" in kwargs:
            return super().__new__(cls, stream_id=kwargs["stream_id"], device_index=kwargs["device_index"],
                                   device_type=kwargs["device_type"])
        import torch_gcu.gcu as gcu
        gcu._lazy_init()
        if device is None:
            device = torch.device("gcu", gcu.current_device())
        elif isinstance(device, int):
            device = torch.device("gcu", device)
        else:
            device = torch.device(device)
            if device.index is None:
                device = torch.device("gcu", gcu.current_device())
        return super().__new__(cls, device=device, priority=priority)

    @property
    def gcu_stream(self) -> int:
        """The raw stream handle (a cudaStream_t as an integer; 0 is the default stream)."""
        return _C._gcu_streamHandle(self.stream_id, self.device_index)

    cuda_stream = gcu_stream
    _as_parameter_ = gcu_stream

    @property
    def priority(self) -> int:
        return -1 if 32 < self.stream_id <= 64 else 0

    @staticmethod
    def priority_range():
        return _C._gcu_streamPriorityRange()

    def wait_stream(self, stream) -> None:
        self.wait_event(stream.record_event())

    def wait_event(self, event) -> None:
        super().wait_event(event._ev if isinstance(event, Event) else event)

    def record_event(self, event=None):
        if event is None:
            event = Event()
        event.record(self)
        return event

    def __repr__(self):
        return "<torch_gcu.gcu.Stream device=%s gcu_stream=%#x>" % (self.device, self.gcu_stream)


class ExternalStream(Stream):
    """Wraps a stream created outside PyTorch (reference: streams.py:121-142)."""

    def __new__(cls, stream_ptr, device=None, **kwargs):
        import torch_gcu.gcu as gcu
        gcu._lazy_init()
        idx = gcu._get_device_index(device)
        sid, didx, dtype = _C._gcu_getStreamFromExternal(int(stream_ptr), idx)
        return super().__new__(cls, stream_id=sid, device_index=didx, device_type=dtype)


class Event:
    """Event(enable_timing=False, blocking=False, interprocess=False) with record / wait /
    query / elapsed_time / synchronize (reference: streams.py:144-237). It wraps the
    device-generic torch.Event, which the device guard implements."""

    def __init__(self, enable_timing=False, blocking=False, interprocess=False):
        if interprocess:
            raise NotImplementedError("interprocess events are not supported by the gcu backend")
        self._ev = torch.Event(device="gcu", enable_timing=enable_timing)

    def record(self, stream=None):
        if stream is None:
            import torch_gcu.gcu as gcu
            stream = gcu.current_stream()
        self._ev.record(stream)

    def wait(self, stream=None) -> None:
        if stream is None:
            import torch_gcu.gcu as gcu
            stream = gcu.current_stream()
        self._ev.wait(stream)

    def query(self) -> bool:
        return self._ev.query()

    def elapsed_time(self, end_event) -> float:
        return self._ev.elapsed_time(end_event._ev if isinstance(end_event, Event) else end_event)

    def synchronize(self) -> None:
        self._ev.synchronize()

    @property
    def device(self):
        return self._ev.device
