"""Needle-in-a-haystack evaluation: the NIAH subset of scripts/eval_ruler.py with its defaults
(reference scripts/eval_niah.py: tasks niah_*, 128 new tokens)."""
import sys

from eval_ruler import main

if __name__ == "__main__":
    argv = sys.argv[1:]
    if "--tasks" not in argv:
        argv += ["--tasks", "niah_single_1", "niah_single_2", "niah_single_3", "niah_multikey_1", "niah_multikey_2",
                 "niah_multikey_3", "niah_multivalue", "niah_multiquery"]
    main(argv)
