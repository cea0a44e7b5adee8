/* Stand-in for the reference's src/nextdoor.cu when its example app is compiled for the host:
 * the shim header included before it already declares everything an App body needs. */
