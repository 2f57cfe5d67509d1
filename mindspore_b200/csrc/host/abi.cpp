extern "C" __attribute__((visibility("default"))) int msb_host_abi_version() { return 2; }
