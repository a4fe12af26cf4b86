"""SO-101 arm support: Feetech serial bus, cameras, follower / leader devices and the command-line tools
(reference ``src/opentau/scripts/so101/**``).  Pure host-side I/O; nothing here touches a GPU."""
