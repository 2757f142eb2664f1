// Stand-in for <systemd/sd-bus.h> (libsystemd headers are not installed). The shutdown-capture class only
// needs the type names to be declared; nothing on the training step calls into it.
#pragma once
struct sd_bus;
struct sd_bus_message;
struct sd_bus_error { const char *name; const char *message; int _need_free; };
#define SD_BUS_ERROR_NULL {nullptr, nullptr, 0}
