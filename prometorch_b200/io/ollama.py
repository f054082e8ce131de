"""Resolve Ollama model names to GGUF blobs: ``~/.ollama/models/manifests/registry.ollama.ai/library/<name>/<tag>``
lists layers; the layer with media type ``application/vnd.ollama.image.model`` names the blob
``blobs/sha256-<hex>`` (torch/io/ollama.h:30-208).  ``OLLAMA_MODELS`` overrides the root.  A direct path
to a ``.gguf`` file is accepted everywhere a model name is."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional


def models_root() -> str:
    return os.environ.get("OLLAMA_MODELS", os.path.join(os.path.expanduser("~"), ".ollama", "models"))


def resolve_model(name: str, root: Optional[str] = None) -> str:
    if os.path.isfile(name):
        return name
    root = root or models_root()
    model, _, tag = name.partition(":")
    tag = tag or "latest"
    manifest = os.path.join(root, "manifests", "registry.ollama.ai", "library", model, tag)
    if not os.path.isfile(manifest):
        raise FileNotFoundError(f"model '{name}' not found (looked for {manifest})")
    with open(manifest) as f:
        m = json.load(f)
    for layer in m.get("layers", []):
        if layer.get("mediaType", "").endswith("image.model"):
            blob = os.path.join(root, "blobs", layer["digest"].replace(":", "-"))
            if os.path.isfile(blob):
                return blob
            raise FileNotFoundError(f"blob for '{name}' is missing: {blob}")
    raise FileNotFoundError(f"manifest of '{name}' has no model layer")


def list_models(root: Optional[str] = None, extra_dirs: Optional[List[str]] = None) -> List[Dict]:
    """Installed models as ``{name, path, size, modified}`` (Ollama store plus any ``.gguf`` in ``extra_dirs``)."""
    out = []
    root = root or models_root()
    lib = os.path.join(root, "manifests", "registry.ollama.ai", "library")
    if os.path.isdir(lib):
        for model in sorted(os.listdir(lib)):
            for tag in sorted(os.listdir(os.path.join(lib, model))):
                try:
                    p = resolve_model(f"{model}:{tag}", root)
                    st = os.stat(p)
                    out.append({"name": f"{model}:{tag}", "path": p, "size": st.st_size, "modified": st.st_mtime})
                except (FileNotFoundError, json.JSONDecodeError, KeyError):
                    continue
    for d in extra_dirs or []:
        if os.path.isdir(d):
            for fn in sorted(os.listdir(d)):
                if fn.endswith(".gguf"):
                    p = os.path.join(d, fn)
                    st = os.stat(p)
                    out.append({"name": fn[:-5], "path": p, "size": st.st_size, "modified": st.st_mtime})
    return out
