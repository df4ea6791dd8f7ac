"""B200-native backend for the decoder-block hot path of the reference C++
training engine.  The package directory name is not a Python identifier;
import it with ``importlib.import_module("large-language-model_b200")``.
"""
