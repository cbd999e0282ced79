"""Builders: configuration objects that assemble an encoder whose attention is picked from
the registry by name.

Mirror of ``fast_transformers/builders`` for the encoder path: ``BaseBuilder``
(``base.py:10-67``), ``AttentionBuilder`` / ``RecurrentAttentionBuilder``
(``attention_builders.py:15-130``), ``TransformerEncoderBuilder`` and ``RecurrentEncoderBuilder``
(``transformer_builders.py:24-320``; same parameters, the recurrent one assembles the
one-position-at-a-time classes from the recurrent registry).  Kept behaviours:
attribute-style parameters; unknown keys raise ``ValueError`` from ``from_kwargs`` /
``from_dictionary`` unless ``strict=False`` (``from_namespace`` defaults to non-strict);
attributes that are not builder properties are forwarded to the attention builder, which
validates them against the registry; composition strings ``"outer:inner1,inner2"``.
Defaults: 4 layers, 4 heads, 64/64 query/value dims, FFN 1024, dropout 0.1, relu, final
LayerNorm, ``attention_type="full"`` -- which is not registered in this package, so
``attention_type`` must be set (to ``"causal-linear"``) before ``get()``.
"""
from collections import defaultdict

from torch.nn import LayerNorm

from ..attention import AttentionLayer
from ..attention_registry import AttentionRegistry, RecurrentAttentionRegistry
from ..recurrent.attention import RecurrentAttentionLayer
from ..recurrent.transformers import (RecurrentTransformerEncoder,
                                      RecurrentTransformerEncoderLayer)
from ..transformers import TransformerEncoder, TransformerEncoderLayer


class BaseBuilder(object):
    @classmethod
    def from_kwargs(cls, **kwargs):
        strict = kwargs.pop("strict", True)
        return cls.from_dictionary(kwargs, strict=strict)

    @classmethod
    def from_namespace(cls, args, strict=False):
        return cls.from_dictionary(vars(args), strict=strict)

    @classmethod
    def from_dictionary(cls, dictionary, strict=True):
        builder = cls()
        for key, value in dictionary.items():
            try:
                setattr(builder, key, value)
            except AttributeError:
                if strict:
                    raise ValueError("The builder has no parameter {!r}".format(key))
        return builder


class BaseAttentionBuilder(BaseBuilder):
    def __init__(self, registry):
        self._registry = registry
        self._parameters = defaultdict(lambda: None)

    @property
    def available_attentions(self):
        return self._registry.keys

    def validate_attention_type(self, attention_type):
        return all(all(t in self._registry for t in a.split(","))
                   for a in attention_type.split(":"))

    def __setattr__(self, key, value):
        if key in ("_registry", "_parameters"):
            return object.__setattr__(self, key, value)
        if not self._registry.contains_parameter(key):
            raise AttributeError("{!r} is not a valid attention parameter name".format(key))
        self._parameters[key] = self._registry.validate_parameter(key, value)

    def __getattr__(self, key):
        if key in self._parameters:
            return self._parameters[key]
        raise AttributeError()

    def __repr__(self):
        body = "\n".join("    {}={!r},".format(k, v) for k, v in self._parameters.items())
        return "{}.from_kwargs(\n{}\n)".format(self.__class__.__name__, body[:-1])

    def get(self, attention_type):
        """Instantiate ``attention_type``; ``"a:b,c"`` builds b and c and passes them to a."""
        attentions = []
        for level in reversed(attention_type.split(":")):
            attentions = [self._construct_attention(t, attentions) for t in level.split(",")]
        if len(attentions) > 1:
            raise ValueError("Invalid attention_type argument {!r}".format(attention_type))
        return attentions[0]

    def _construct_attention(self, attention_type, decorated=()):
        if attention_type not in self._registry:
            raise ValueError("Unknown attention type {!r}".format(attention_type))
        attention, parameters = self._registry[attention_type]
        kwargs = {p: self._registry.validate_parameter(p, self._parameters[p])
                  for p in parameters}
        return attention(*decorated, **kwargs)


class AttentionBuilder(BaseAttentionBuilder):
    def __init__(self):
        super().__init__(AttentionRegistry)


class RecurrentAttentionBuilder(BaseAttentionBuilder):
    def __init__(self):
        super().__init__(RecurrentAttentionRegistry)


class TransformerEncoderBuilder(BaseBuilder):
    """``TransformerEncoderBuilder.from_kwargs(n_layers=..., attention_type="causal-linear",
    ...).get()`` returns a ``TransformerEncoder``."""

    _PROPERTIES = ("n_layers", "n_heads", "feed_forward_dimensions", "query_dimensions",
                   "value_dimensions", "model_dimensions", "dropout", "activation",
                   "final_normalization", "event_dispatcher", "attention_type")
    # what get() assembles (transformer_builders.py:166-181: the _get_*_class hooks)
    _ATTENTION_BUILDER = AttentionBuilder
    _ATTENTION_LAYER = AttentionLayer
    _ENCODER_LAYER = TransformerEncoderLayer
    _ENCODER = TransformerEncoder

    def __init__(self):
        self._n_layers = 4
        self._n_heads = 4
        self._d_query = 64
        self._d_value = 64
        self._d_ff = 1024
        self._d_model = None
        self._dropout = 0.1
        self._activation = "relu"
        self._final_norm = True
        self._event_dispatcher = ""
        self._attention_builder = self._ATTENTION_BUILDER()
        self._attention_type = "full"

    # plain parameters -----------------------------------------------------------------
    n_layers = property(lambda s: s._n_layers, lambda s, v: s._set("_n_layers", v))
    n_heads = property(lambda s: s._n_heads, lambda s, v: s._set("_n_heads", v))
    feed_forward_dimensions = property(lambda s: s._d_ff, lambda s, v: s._set("_d_ff", v))
    query_dimensions = property(lambda s: s._d_query, lambda s, v: s._set("_d_query", v))
    value_dimensions = property(lambda s: s._d_value, lambda s, v: s._set("_d_value", v))
    dropout = property(lambda s: s._dropout, lambda s, v: s._set("_dropout", v))
    event_dispatcher = property(lambda s: s._event_dispatcher,
                                lambda s, v: s._set("_event_dispatcher", v))

    def _set(self, name, value):
        object.__setattr__(self, name, value)

    @property
    def model_dimensions(self):
        return self._d_model or self.value_dimensions * self.n_heads

    @model_dimensions.setter
    def model_dimensions(self, n):
        self._d_model = n

    @property
    def activation(self):
        return self._activation

    @activation.setter
    def activation(self, val):
        activations = ["relu", "gelu"]
        if val not in activations:
            raise ValueError("{!r} is not one of the available activation types {!r}".format(
                val, activations))
        self._activation = val

    @property
    def final_normalization(self):
        return self._final_norm

    @final_normalization.setter
    def final_normalization(self, val):
        self._final_norm = bool(val)

    @property
    def attention(self):
        """The attention builder; its parameters can also be set on this object."""
        return self._attention_builder

    @property
    def attention_type(self):
        return self._attention_type

    @attention_type.setter
    def attention_type(self, val):
        if not self._attention_builder.validate_attention_type(val):
            raise ValueError("{!r} is not an available attention type".format(val))
        self._attention_type = val

    def __setattr__(self, key, val):
        if key[0] == "_":
            return object.__setattr__(self, key, val)
        # own properties are set here; the same name may also be an attention parameter
        # (query_dimensions, event_dispatcher), so it is offered to the attention builder too
        own = key in self._PROPERTIES or hasattr(self, key)
        if own:
            object.__setattr__(self, key, val)
        try:
            setattr(self._attention_builder, key, val)
        except Exception:
            if not own:
                raise

    def get(self):
        self.attention.event_dispatcher = self.event_dispatcher
        d_model = self.model_dimensions
        layers = [
            self._ENCODER_LAYER(
                self._ATTENTION_LAYER(
                    self.attention.get(self.attention_type), d_model, self.n_heads,
                    d_keys=self.query_dimensions, d_values=self.value_dimensions,
                    event_dispatcher=self.event_dispatcher),
                d_model, self.feed_forward_dimensions, self.dropout, self.activation,
                event_dispatcher=self.event_dispatcher)
            for _ in range(self.n_layers)
        ]
        norm = LayerNorm(d_model) if self.final_normalization else None
        return self._ENCODER(layers, norm, event_dispatcher=self.event_dispatcher)


class RecurrentEncoderBuilder(TransformerEncoderBuilder):
    """``RecurrentEncoderBuilder.from_kwargs(attention_type="causal-linear", ...).get()`` returns a
    ``RecurrentTransformerEncoder``: the same parameters and the same weights as the batch
    encoder (``load_state_dict`` of one into the other), evaluated one position at a time
    (``transformer_builders.py:289-320``)."""

    _ATTENTION_BUILDER = RecurrentAttentionBuilder
    _ATTENTION_LAYER = RecurrentAttentionLayer
    _ENCODER_LAYER = RecurrentTransformerEncoderLayer
    _ENCODER = RecurrentTransformerEncoder
