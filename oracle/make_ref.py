"""Put the reference's own model code where the tests and the benchmark's CPU leg can import it without the reference's
checkout: oracle/_ref/models/{llama,gpt2}.py, copied unmodified from the checkout given (default: the path in
$FERRITE_REFERENCE, else /root/reference), and a two-line package oracle/_ref/ferrite/ whose `tensor` module is
ferrite_b200's - the import the reference's models make (`from ferrite.tensor import Tensor, jit`, models/llama.py:20,
models/gpt2.py:12) then binds this library's Tensor.  TEST INFRASTRUCTURE ONLY; oracle/_ref/ is not part of the
repository's history (it is rebuilt from a checkout by this script, which `__graft_entry__.build()` runs when a checkout
is there), and nothing under ferrite_b200/ reads it.

    python oracle/make_ref.py [path/to/reference]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIM = '''"""`ferrite.tensor` for the reference's models: this library's Tensor, jit and Runtime (oracle/make_ref.py wrote this file)."""
from ferrite_b200.tensor import Runtime, Tensor, jit  # noqa: F401
'''


def make(checkout=None):
    checkout = checkout or os.environ.get("FERRITE_REFERENCE", "/root/reference")
    models = os.path.join(checkout, "models")
    if not os.path.isfile(os.path.join(models, "llama.py")):
        return None
    os.makedirs(os.path.join(REF, "models"), exist_ok=True)
    os.makedirs(os.path.join(REF, "ferrite"), exist_ok=True)
    for name in ("llama.py", "gpt2.py"):
        shutil.copyfile(os.path.join(models, name), os.path.join(REF, "models", name))
    with open(os.path.join(REF, "ferrite", "__init__.py"), "w") as f:
        f.write('"""Stands in for the reference\'s package on the import path of its models (oracle/make_ref.py)."""\n')
    with open(os.path.join(REF, "ferrite", "tensor.py"), "w") as f:
        f.write(SHIM)
    return REF


def modules():
    """(llama, gpt2): the reference's model modules from oracle/_ref, bound to ferrite_b200's Tensor; None if absent."""
    if not os.path.isfile(os.path.join(REF, "models", "llama.py")):
        return None
    import importlib.util
    root = os.path.dirname(HERE)
    for p in (root, REF, os.path.join(REF, "models")):
        if p not in sys.path:
            sys.path.insert(0, p)
    loaded = []
    for name in ("gpt2", "llama"):  # (gpt2 first: llama imports it by that name)
        key = name if name == "gpt2" else "reference_llama"
        if key not in sys.modules:
            spec = importlib.util.spec_from_file_location(key, os.path.join(REF, "models", name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[key] = mod
            spec.loader.exec_module(mod)
        loaded.append(sys.modules[key])
    return loaded[1], loaded[0]


if __name__ == "__main__":
    print(make(sys.argv[1] if len(sys.argv) > 1 else None) or "no reference checkout found")
