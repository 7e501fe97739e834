"""CPU oracle for the NVFP4 path. Test infrastructure only: nothing shipped imports it."""
