"""Sphinx configuration for the kempnerforge_b200 documentation (Markdown pages through MyST; API pages from docstrings).

    pip install sphinx myst-parser furo
    sphinx-build -b html docs docs/_build/html
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.abspath(".."))

project = "kempnerforge_b200"
author = "kempnerforge_b200 contributors"
release = "0.2.0"

extensions = ["sphinx.ext.autodoc", "sphinx.ext.autosummary", "sphinx.ext.napoleon", "sphinx.ext.viewcode", "myst_parser"]
source_suffix = {".rst": "restructuredtext", ".md": "markdown"}
exclude_patterns = ["_build"]
autosummary_generate = True
# the API pages are built on machines without a GPU or the heavy dependencies
autodoc_mock_imports = ["torch", "numpy", "transformers", "datasets", "wandb", "tensorboard", "pyarrow", "sentencepiece", "PIL"]
autodoc_default_options = {"members": True, "show-inheritance": True, "member-order": "bysource"}
myst_enable_extensions = ["colon_fence", "deflist"]
html_theme = "furo"
html_title = "kempnerforge_b200"
