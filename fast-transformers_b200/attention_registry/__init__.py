"""The plugin table that maps an attention name to its class and constructor parameters.

Mirror of ``fast_transformers/attention_registry`` (``registry.py:7-59``, ``spec.py:12-126``)
restricted to what the ``"causal-linear"`` entry and the attention builder use.  Behaviour
kept: duplicate keys raise ``ValueError`` (registry.py:17-18); a parameter re-registered with
a different Spec raises (:22-33); ``validate_parameter`` wraps any failure in ``ValueError``
(:51-56).
"""
from ..events import EventDispatcher


class Spec(object):
    """Validator/canonicaliser of one constructor parameter."""

    def __init__(self, predicate, name="CustomSpec"):
        self._predicate = predicate
        self._name = name

    def __repr__(self):
        return self._name

    def get(self, x):
        return self._predicate(x)

    def check(self, x):
        try:
            self.get(x)
            return True
        except ValueError:
            return False

    def __eq__(self, other):
        return self is other

    __hash__ = object.__hash__


class Choice(Spec):
    def __init__(self, choices):
        self._choices = choices

    def get(self, x):
        if x in self._choices:
            return x
        raise ValueError("{!r} is not in {!r}".format(x, self._choices))

    def __repr__(self):
        return "Choice({!r})".format(self._choices)

    def __eq__(self, other):
        return isinstance(other, Choice) and self._choices == other._choices

    __hash__ = object.__hash__


class Optional(Spec):
    """A parameter that may be None, in which case ``default`` is used."""

    def __init__(self, spec, default=None):
        self._other_spec = spec
        self._default = default

    def __repr__(self):
        return "Optional[{!r}, {!r}]".format(self._other_spec, self._default)

    def get(self, x):
        return self._default if x is None else self._other_spec.get(x)

    def __eq__(self, other):
        return (isinstance(other, Optional) and self._other_spec == other._other_spec
                and self._default == other._default)

    __hash__ = object.__hash__


def _callable(x):
    if callable(x):
        return x
    raise ValueError("{!r} is not a callable".format(x))


def _dispatcher(x):
    if isinstance(x, (str, EventDispatcher)):
        return x
    raise ValueError("{!r} is not an event dispatcher".format(x))


Int = Spec(int, "Int")
Float = Spec(float, "Float")
Bool = Spec(bool, "Bool")
Callable = Spec(_callable, "Callable")
EventDispatcherInstance = Spec(_dispatcher, "EventDispatcherInstance")


class Registry(object):
    def __init__(self):
        self._classes = {}
        self._class_params = {}
        self._parameters = {}

    def register(self, key, class_object, parameter_tuples):
        if key in self._classes:
            raise ValueError("{} is already registered".format(key))
        for name, spec in parameter_tuples:
            known = self._parameters.get(name)
            if known is not None and known != spec:
                raise ValueError("{} is already registered with spec {!r} instead of {!r}".format(
                    name, known, spec))
        self._classes[key] = class_object
        for name, spec in parameter_tuples:
            self._parameters[name] = spec
        self._class_params[key] = [name for name, _ in parameter_tuples]

    def __contains__(self, key):
        return key in self._classes

    def __getitem__(self, key):
        return self._classes[key], self._class_params[key]

    @property
    def keys(self):
        return list(self._classes.keys())

    def contains_parameter(self, key):
        return key in self._parameters

    def validate_parameter(self, key, value):
        try:
            return self._parameters[key].get(value)
        except Exception as e:
            raise ValueError("Invalid value {!r} for parameter {!r}".format(value, key)) from e


AttentionRegistry = Registry()
# attention implementations that process one position at a time and carry a state
# (fast_transformers/attention_registry/__init__.py:12-15)
RecurrentAttentionRegistry = Registry()
# attention over a fixed memory, one query per call (same file, :16)
RecurrentCrossAttentionRegistry = Registry()
