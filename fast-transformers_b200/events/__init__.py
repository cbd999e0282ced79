"""Observer hooks used by the attention layer and the encoder (host-side only).

Mirror of the part of ``fast_transformers/events`` that the causal-linear path touches:
``EventDispatcher`` (``events/event_dispatcher.py:12-92``) and the event payload classes
(``events/event.py:7-65``).  Filters are plain callables ``event -> bool``; passing an Event
subclass to ``listen`` filters by type.
"""
from collections import OrderedDict


class Event(object):
    """Base event: remembers the module that emitted it."""

    def __init__(self, source):
        self.source = source


class AttentionEvent(Event):
    def __init__(self, source, attention_matrix):
        super().__init__(source)
        self.attention_matrix = attention_matrix


class QKVEvent(Event):
    """Projected queries (N, L, H, E), keys (N, S, H, E) and values (N, S, H, D)."""

    def __init__(self, source, queries, keys, values):
        super().__init__(source)
        self.queries = queries
        self.keys = keys
        self.values = values


class IntermediateOutput(Event):
    """Output (N, L, D) of one encoder layer."""

    def __init__(self, source, x):
        super().__init__(source)
        self.x = x


class EventDispatcher(object):
    """Named, process-global dispatchers; ``get("")`` is the default one."""
    _dispatchers = {}

    def __init__(self):
        self._listeners = OrderedDict()

    def listen(self, event_filter, event_handler):
        if isinstance(event_filter, type) and issubclass(event_filter, Event):
            cls = event_filter
            event_filter = lambda ev, _c=cls: isinstance(ev, _c)  # noqa: E731
        self._listeners[event_handler] = event_filter

    def remove(self, event_handler):
        self._listeners.pop(event_handler, None)

    def clear(self):
        self._listeners.clear()

    def dispatch(self, event):
        for handler, accepts in self._listeners.items():
            if accepts(event):
                handler(event)

    @classmethod
    def get(cls, key=""):
        if isinstance(key, cls):
            return key
        if key not in cls._dispatchers:
            cls._dispatchers[key] = cls()
        return cls._dispatchers[key]
