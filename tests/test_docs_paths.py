"""The notes cite files of this repository by path; a citation of a file that is not there is a stale note."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_repository_path_the_notes_cite_exists():
    missing = []
    for doc in ("DESIGN.md", "INTEGRATION.md", "README.md", "BASELINE.md"):
        text = open(os.path.join(ROOT, doc)).read()
        for path in set(re.findall(r"`((?:profiles|tests|oracle|include|oxidizr_b200)/[A-Za-z0-9_./-]+?)`", text)):
            path = path.split("::")[0].rstrip("/")
            if "*" in path or path.endswith("...") or path == "oracle/_ref":  # the latter is cited as what cannot exist here
                continue
            if not os.path.exists(os.path.join(ROOT, path)) and not path.endswith(".so"):
                missing.append((doc, path))
    assert not missing, missing
