"""Known public protein datasets (key -> download URL), same keys as the reference
(src/nanoplm/config/datasets.py:13-24)."""
from __future__ import annotations

_UNIPROT = "https://ftp.uniprot.org/pub/databases/uniprot"

DATASET_URLS: dict[str, str] = {
    "swissprot": f"{_UNIPROT}/knowledgebase/complete/uniprot_sprot.fasta.gz",
    "trembl": f"{_UNIPROT}/knowledgebase/complete/uniprot_trembl.fasta.gz",
    "uniref50": f"{_UNIPROT}/uniref/uniref50/uniref50.fasta.gz",
    "uniref90": f"{_UNIPROT}/uniref/uniref90/uniref90.fasta.gz",
    "uniref100": f"{_UNIPROT}/uniref/uniref100/uniref100.fasta.gz",
}


def get_supported_datasets() -> dict[str, str]:
    return dict(DATASET_URLS)


def resolve_dataset_url(key_or_none: str | None, url: str | None) -> str:
    if url:
        return url
    if key_or_none is None:
        raise KeyError("either a dataset key or --url is required")
    k = key_or_none.lower()
    if k not in DATASET_URLS:
        raise KeyError(f"Unknown dataset '{key_or_none}'. Known: {', '.join(sorted(DATASET_URLS))}")
    return DATASET_URLS[k]
