"""TEST INFRASTRUCTURE: CPU oracle for the kernel set (see oracle.c and oracle/oracle.py)."""
