"""Prints interpreter / torch / CUDA / GPU facts (reference ``src/opentau/scripts/display_sys_info.py``)."""

from ..utils.utils import display_sys_info

if __name__ == "__main__":
    display_sys_info()
