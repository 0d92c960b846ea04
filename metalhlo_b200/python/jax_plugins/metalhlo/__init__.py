"""JAX entry point of the B200 backend: registers ``pjrt_plugin_metalhlo_b200.so`` as the PJRT plugin "metalhlo".

JAX discovers plugins through the ``jax_plugins`` namespace package: put the directory that holds this ``jax_plugins``
folder on ``PYTHONPATH`` (``metalhlo_b200/python``) and ``jax.devices("metalhlo")`` lists the GPUs the plugin exposes
(one by default, ``METALHLO_NUM_GPUS`` of them when set). Same role as the reference's
``python/jax_plugins/metalhlo/__init__.py:13-69``; the plugin name stays "metalhlo" so that user code written against
the reference selects this backend unchanged.

jax / jaxlib are imported inside ``initialize()`` only, so that the module (and its helpers) import without them.
"""
import os
import sys

PLUGIN_NAME = "metalhlo"
_HERE = os.path.dirname(os.path.abspath(__file__))


def plugin_candidates():
    """Paths where the plugin library is looked for, in order: METALHLO_PLUGIN_PATH, beside this package (a wheel), and
    the in-tree build directory."""
    out = []
    env_path = os.environ.get("METALHLO_PLUGIN_PATH")
    if env_path:
        out.append(env_path)
    out.append(os.path.join(_HERE, "pjrt_plugin_metalhlo_b200.so"))
    out.append(os.path.join(_HERE, "..", "..", "..", "lib", "pjrt_plugin_metalhlo_b200.so"))
    return out


def find_plugin():
    for path in plugin_candidates():
        resolved = os.path.realpath(path)
        if os.path.isfile(resolved):
            return resolved
    raise RuntimeError("Could not find pjrt_plugin_metalhlo_b200.so. Build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                       "or set METALHLO_PLUGIN_PATH to the library.")


def prepare_environment():
    """What the plugin's bytecode helper needs: the interpreter that has jaxlib, and the helper script. Both can be
    overridden by the caller; defaults are this interpreter and the script beside this file."""
    os.environ.setdefault("METALHLO_PYTHON", sys.executable)
    os.environ.setdefault("METALHLO_BYTECODE_HELPER", os.path.join(_HERE, "bytecode_to_text.py"))


def initialize():
    """Register the plugin with JAX's PJRT backend system (called by JAX's plugin discovery)."""
    prepare_environment()
    import jax._src.xla_bridge as xb
    import jaxlib.xla_client as xla_client

    # newer JAX rejects a second registration of a loaded plugin with ALREADY_EXISTS
    loaded = getattr(xla_client, "pjrt_plugin_loaded", None)
    if loaded is not None and loaded(PLUGIN_NAME):
        return
    xb.register_plugin(PLUGIN_NAME, priority=500, library_path=find_plugin(), options=None)
