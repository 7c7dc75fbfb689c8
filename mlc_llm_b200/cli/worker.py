"""``python -m mlc_llm_b200.cli.worker``: one tensor-/pipeline-parallel worker rank (reference:
``python/mlc_llm/cli/worker.py``)."""
from ..parallel.launcher import worker_main


def main(argv=None):
    worker_main(argv)


if __name__ == "__main__":
    main()
