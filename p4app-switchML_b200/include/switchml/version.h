// Version banner printed when the context is created (reference context.cc:51-53 prints
// the git hash and the build flags injected by client_lib/Makefile:154-159).
#ifndef SWITCHML_VERSION_H_
#define SWITCHML_VERSION_H_

#define SWITCHML_VERSION "0.1.0"
#ifndef SWITCHML_BUILD_INFO
#define SWITCHML_BUILD_INFO "sm_100a; backends: dummy udp cuda"
#endif

#endif  // SWITCHML_VERSION_H_
