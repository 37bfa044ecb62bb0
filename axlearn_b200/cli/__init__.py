"""Command line: ``python -m axlearn_b200.cli <group> <command> ...``.

Parity target in the reference: axlearn/cli/__init__.py and axlearn/cli/utils.py (an absl command
tree ``axlearn <group> <cmd>``; the gcp group launches through the bastion).  Groups here:

* ``train``      run a named trainer config (``common.launch_trainer``);
* ``bench``      the repository's benchmark entry point;
* ``bastion``    ``start | submit | cancel | list | state`` against a bastion directory;
* ``bundle``     tar the source tree into a bundle directory.
"""
