"""State handling shared by the recurrent modules (``fast_transformers/recurrent/_utils.py``)."""
import warnings


def check_state(state=None, memory=None):
    """``memory`` is the deprecated name of ``state`` (``_utils.py:9-16``)."""
    if memory is not None:
        warnings.warn("'memory' is deprecated for recurrent transformers and will be removed in "
                      "the future, use 'state' instead", DeprecationWarning)
    if state is None:
        state = memory
    return state
