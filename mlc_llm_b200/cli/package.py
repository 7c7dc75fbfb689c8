"""``mlc_llm_b200 package``: bundling model libraries and weights into iOS / Android app projects
(reference: ``python/mlc_llm/interface/package.py``) targets mobile back ends that this sm_100a
build does not have; the command explains that and exits non-zero."""
import sys


def main(argv=None):
    _ = argv
    print("package: mobile (iOS / Android) targets are not part of this build; "
          "serve converted weights with `python -m mlc_llm_b200 serve` instead.", file=sys.stderr)
    sys.exit(1)


if __name__ == "__main__":
    main()
