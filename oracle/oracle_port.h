/* TEST INFRASTRUCTURE - declarations of the plain-C restatement (oracle/ *_port.c). */
#ifndef ORACLE_PORT_H
#define ORACLE_PORT_H
#include <stddef.h>
#include <stdint.h>
#endif
