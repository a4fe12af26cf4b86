"""``opentau-so101-find-port``: unplug the arm when asked; the serial device that disappears is its port."""

import glob
import time

from .device_paths import stable_serial_path


def list_ports() -> set[str]:
    return set(glob.glob("/dev/ttyACM*") + glob.glob("/dev/ttyUSB*") + glob.glob("/dev/tty.usbmodem*"))


def main(argv=None):
    import argparse
    argparse.ArgumentParser(description=__doc__).parse_args(argv)        # no options: --help explains the procedure
    before = list_ports()
    input("Unplug the USB cable of the arm and press Enter...")
    time.sleep(0.5)
    gone = before - list_ports()
    if len(gone) == 1:
        port = gone.pop()
        print(f"The port of this arm is {port}. Plug the cable back in.")
        input("Press Enter once it is plugged in again...")
        stable = stable_serial_path(port)
        if stable:
            print(f"Use the stable name in configs (it survives reboots and replugs): {stable}")
    else:
        print(f"Could not identify the port (candidates: {sorted(gone) or 'none'}).")


if __name__ == "__main__":
    main()
