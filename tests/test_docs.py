"""The committed API reference covers the live package (regenerate with `python -m mscclpp_b200.utils.apidoc`)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_api_reference_names_every_public_symbol():
    import mscclpp_b200 as mp

    text = open(os.path.join(ROOT, "docs", "api-reference.md")).read()
    missing = [n for n in mp.__all__ if not n.startswith("__") and f"`{n}" not in text]
    assert not missing, f"docs/api-reference.md is stale, missing: {missing}"
    native = mp.native()
    public = [n for n in dir(native) if not n.startswith("_")]
    missing = [n for n in public if f"`{n}" not in text]
    assert not missing, f"docs/api-reference.md is stale, native names missing: {missing}"
    # every public header is listed
    inc = os.path.join(ROOT, "mscclpp_b200", "csrc", "include", "mscclpp")
    headers = [f for f in os.listdir(inc) if f.endswith(".hpp")]
    missing = [h for h in headers if f"<mscclpp/{h}>" not in text]
    assert not missing, missing


def test_guides_link_to_existing_files():
    docs = os.path.join(ROOT, "docs")
    for name in os.listdir(docs):
        if not name.endswith(".md"):
            continue
        for target in re.findall(r"\]\(([^)#]+\.md)\)", open(os.path.join(docs, name)).read()):
            assert os.path.exists(os.path.normpath(os.path.join(docs, target))), (name, target)
