"""Child of tests/test_launchers.py: the first incarnation of a group waits to be hit by an injected failure, every
later one exits successfully.  Incarnations are counted in a file named by the environment."""
import os
import sys
import time

path = os.path.join(os.environ["SLEEPY_DIR"], f"group{os.environ['REPLICA_GROUP_ID']}.count")
with open(path, "a") as f:
    f.write("x\n")
with open(path) as f:
    incarnation = len(f.read().splitlines())
print(f"incarnation {incarnation}", flush=True)
if incarnation >= 2:
    sys.exit(0)
time.sleep(600)
