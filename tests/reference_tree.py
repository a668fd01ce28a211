"""Where the tests find a checkout of the reference project (violetDelia/LLCompiler), whose lit files some of them
read: the directory named by LLC_REFERENCE_ROOT, else a directory called `reference` beside this repository.
Tests that need it skip when neither exists; nothing of the reference is copied into this tree."""
import os

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_root():
    for cand in (os.environ.get("LLC_REFERENCE_ROOT"), os.path.join(os.path.dirname(_ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "test", "Dialect", "LLH")):
            return cand
    return None


def reference_path(*parts):
    root = reference_root()
    return os.path.join(root, *parts) if root else None
