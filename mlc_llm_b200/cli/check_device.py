"""``mlc_llm_b200 check_device <kind>``: print the device indices of that kind, one line, or nothing
(reference: ``python/mlc_llm/cli/check_device.py``)."""
import sys

import torch


def main(argv=None):
    argv = argv if argv is not None else sys.argv[1:]
    kind = argv[0] if argv else "cuda"
    if kind == "cuda" and torch.cuda.is_available():
        print("check_device:" + ",".join(str(i) for i in range(torch.cuda.device_count())))
    elif kind == "cpu":
        print("check_device:0")
    else:
        print("check_device:")


if __name__ == "__main__":
    main()
