"""Runner jobs: launch a workload and babysit it until it ends (reference: axlearn/cloud/gcp/runners)."""
